#ifndef THUNDERSVM_NUSVR_H
#define THUNDERSVM_NUSVR_H
#include <thundersvm/model/svr.h>

/// nu-SVR (include/thundersvm/model/nusvr.h)
class NuSVR : public SVR {
public:
    void train(const DataSet &dataset, SvmParam param) override;
    ~NuSVR() override = default;

protected:
    void model_setup(const DataSet &dataset, SvmParam &param) override;
};
#endif
