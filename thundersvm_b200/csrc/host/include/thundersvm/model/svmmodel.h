// SvmModel: the reference's model base class (include/thundersvm/model/svmmodel.h:18-215): training
// entry point, batched prediction through the kernel matrix of the support vectors, cross
// validation, LibSVM-compatible model text.
#ifndef THUNDERSVM_SVMMODEL_H
#define THUNDERSVM_SVMMODEL_H
#include <thundersvm/dataset.h>
#include <thundersvm/svmparam.h>
#include <thundersvm/kernelmatrix.h>
#include <memory>

class SvmModel {
public:
    virtual void train(const DataSet &dataset, SvmParam param) = 0;
    virtual vector<float_type> predict(const DataSet::node2d &instances, int batch_size);
    virtual vector<float_type> predict_instant(const DataSet::node2d &instances, int batch_size);
    void predict_dec_values(const DataSet::node2d &instances, SyncArray<float_type> &dec_values, int batch_size) const;
    void predict_dec_values_instant(const DataSet::node2d &instances, SyncArray<float_type> &predict_instant,
                                    int batch_size) const;
    virtual vector<float_type> cross_validation(DataSet dataset, SvmParam param, int n_fold);
    virtual void save_to_file(string path);
    virtual void load_from_file(string path);
    virtual string save_to_string();
    virtual void load_from_string(string data);

    int total_sv() const;
    int get_n_classes() const;
    const DataSet::node2d &svs() const;
    const SyncArray<int> &get_n_sv() const;
    const SyncArray<float_type> &get_coef() const;
    const SyncArray<float_type> &get_linear_coef() const;
    const SyncArray<float_type> &get_rho() const;
    void set_max_iter(int iter);
    const SyncArray<float_type> &get_dec_value() const;
    void set_max_memory_size(size_t size);          // MB
    void set_max_memory_size_Byte(size_t size);
    int get_n_binary_models() const;
    const vector<float> &get_prob_predict() const;
    void compute_linear_coef_single_model(size_t n_feature, const bool zero_based);
    void get_param(char *kernel_type, int *degree, float *gamma, float *coef0, int *probability);
    int get_sv_max_index() const;
    const vector<int> &get_sv_ind() const;
    const vector<int> &get_label() const;
    const bool is_prob() const;
    virtual ~SvmModel() = default;

protected:
    virtual void model_setup(const DataSet &dataset, SvmParam &param);
    int get_working_set_size(int n_instances, int n_features);
    /// Kernel matrix of the support vectors, built on the first prediction and kept until the support vectors
    /// change (the reference rebuilds it on every predict call, svmmodel.cpp:84).
    const KernelMatrix &sv_matrix() const;
    void invalidate_sv_matrix() { sv_kmat_.reset(); }

    SvmParam param;
    SyncArray<float_type> coef;
    SyncArray<float_type> linear_coef;
    DataSet::node2d sv;
    vector<int> sv_indices;
    SyncArray<int> n_sv;
    int n_total_sv = 0;
    SyncArray<float_type> rho;
    int n_classes = 2;
    size_t n_binary_models = 1;
    vector<float_type> probA, probB;
    vector<int> label;
    int max_iter = -1;
    SyncArray<float_type> dec_values;
    vector<float> prob_predict;
    int sv_max_index = 0;
    mutable std::unique_ptr<KernelMatrix> sv_kmat_;
};
#endif
