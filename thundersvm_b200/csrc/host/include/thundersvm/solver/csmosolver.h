// CSMOSolver with the reference's public signature (include/thundersvm/solver/csmosolver.h:16-17).
// The reference's protected per-step virtuals (select_working_set, smo_kernel, calculate_rho) are
// folded into the device-resident loop behind tsvm_smo_solve; solver_kind() is the one hook left.
#ifndef THUNDERSVM_CSMOSOLVER_H
#define THUNDERSVM_CSMOSOLVER_H
#include <thundersvm/thundersvm.h>
#include <thundersvm/kernelmatrix.h>

class CSMOSolver {
public:
    void solve(const KernelMatrix &k_mat, const SyncArray<int> &y, SyncArray<float_type> &alpha, float_type &rho,
               SyncArray<float_type> &f_val, float_type eps, float_type Cp, float_type Cn, int ws_size,
               int max_iter) const;
    virtual ~CSMOSolver() = default;

protected:
    virtual int solver_kind() const;     // TSVM_SOLVER_C
};
#endif
