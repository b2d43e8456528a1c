#ifndef THUNDERSVM_SVR_H
#define THUNDERSVM_SVR_H
#include <thundersvm/model/svmmodel.h>

/// epsilon-SVR (include/thundersvm/model/svr.h): the dual over 2n duplicated instances
class SVR : public SvmModel {
public:
    void train(const DataSet &dataset, SvmParam param) override;
    ~SVR() override = default;

protected:
    void model_setup(const DataSet &dataset, SvmParam &param) override;
    void save_svr_coef(const SyncArray<float_type> &alpha_2, const DataSet::node2d &instances);
};
#endif
