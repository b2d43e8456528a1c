// Accuracy / MSE (include/thundersvm/util/metric.h).
#ifndef THUNDERSVM_METRIC_H
#define THUNDERSVM_METRIC_H
#include <thundersvm/thundersvm.h>

class Metric {
public:
    virtual string name() = 0;
    virtual float_type score(const vector<float_type> &predict_y, const vector<float_type> &ground_truth_y) = 0;
    virtual ~Metric() = default;
};
class Accuracy : public Metric {
public:
    string name() override;
    float_type score(const vector<float_type> &predict_y, const vector<float_type> &ground_truth_y) override;
};
class MSE : public Metric {
public:
    string name() override;
    float_type score(const vector<float_type> &predict_y, const vector<float_type> &ground_truth_y) override;
};
#endif
