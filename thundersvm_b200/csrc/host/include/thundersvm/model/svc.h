// C-SVC (include/thundersvm/model/svc.h): one-vs-one over the class pairs, voting or pairwise-coupled
// probabilities at prediction time.
#ifndef THUNDERSVM_SVC_H
#define THUNDERSVM_SVC_H
#include <thundersvm/model/svmmodel.h>

class SVC : public SvmModel {
public:
    void train(const DataSet &dataset, SvmParam param) override;
    vector<float_type> predict(const DataSet::node2d &instances, int batch_size) override;
    vector<float_type> predict_instant(const DataSet::node2d &instances, int batch_size) override;
    ~SVC() override = default;

protected:
    virtual void train_binary(const DataSet &dataset, int i, int j, SyncArray<float_type> &alpha, float_type &rho);
    void model_setup(const DataSet &dataset, SvmParam &param) override;

private:
    vector<float_type> predict_label(const SyncArray<float_type> &dec_values, int n_instances);
    void probability_train(const DataSet &dataset);
    void multiclass_probability(const vector<vector<float_type>> &r, vector<float_type> &p) const;
    vector<float_type> c_weight;

protected:
    // The grouped data set as one dense device matrix, built once per train() when the data qualify for dense
    // storage; the class pairs then take their rows from it on the device.
    struct DeviceRows {
        float *X = nullptr;
        size_t n = 0, d = 0, ld = 0;
    };
    DeviceRows dev_rows_;
    void build_device_rows(const DataSet &grouped);
    void free_device_rows();
};
#endif
