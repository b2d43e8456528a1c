// NuSMOSolver (include/thundersvm/solver/nusmosolver.h:13-16): for_svr = false scales alpha and rho
// (nu-SVC), true leaves them (nu-SVR).
#ifndef THUNDERSVM_NUSMOSOLVER_H
#define THUNDERSVM_NUSMOSOLVER_H
#include "csmosolver.h"

class NuSMOSolver : public CSMOSolver {
public:
    explicit NuSMOSolver(bool for_svr) : for_svr(for_svr) {}
    ~NuSMOSolver() override = default;

protected:
    int solver_kind() const override;

private:
    bool for_svr;
};
#endif
