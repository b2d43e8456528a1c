#ifndef THUNDERSVM_ONECLASS_SVC_H
#define THUNDERSVM_ONECLASS_SVC_H
#include <thundersvm/model/svmmodel.h>

/// one-class SVM (include/thundersvm/model/oneclass_svc.h)
class OneClassSVC : public SvmModel {
public:
    void train(const DataSet &dataset, SvmParam param) override;
    vector<float_type> predict(const DataSet::node2d &instances, int batch_size) override;
    ~OneClassSVC() override = default;

protected:
    void model_setup(const DataSet &dataset, SvmParam &param) override;
};
#endif
