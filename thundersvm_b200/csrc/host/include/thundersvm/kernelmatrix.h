// KernelMatrix with the reference's interface (include/thundersvm/kernelmatrix.h:39-72). The work
// is done on the GPU behind the C ABI (include/thundersvm_b200.h); this class only converts the
// instances once (dense row-major matrix or CSR, chosen by density) and forwards.
#ifndef THUNDERSVM_KERNELMATRIX_H
#define THUNDERSVM_KERNELMATRIX_H
#include "thundersvm.h"
#include "syncarray.h"
#include "dataset.h"
#include "svmparam.h"

struct tsvm_km;

class KernelMatrix {
public:
    explicit KernelMatrix(const DataSet::node2d &instances, SvmParam param);
    /// rows [r0, r0 + n0) followed by rows [r1, r1 + n1) of a dense row-major matrix that is already on the
    /// device (d features, row stride ld floats): the binary sub-problem of two classes of a grouped data set
    /// without a host round trip. No counterpart in the reference, which rebuilds every sub-problem from the
    /// host instances (svc.cpp:147-178).
    KernelMatrix(const float *X_dev, size_t d, size_t ld, size_t r0, size_t n0, size_t r1, size_t n1, SvmParam param);
    ~KernelMatrix();
    KernelMatrix(const KernelMatrix &) = delete;
    KernelMatrix &operator=(const KernelMatrix &) = delete;

    /// rows idx of the kernel matrix: kernel_rows[i * n_instances + j] = K(x_idx[i], x_j)
    void get_rows(const SyncArray<int> &idx, SyncArray<kernel_type> &kernel_rows) const;
    /// kernel values of new instances against the stored ones
    void get_rows(const DataSet::node2d &instances, SyncArray<kernel_type> &kernel_rows) const;
    const SyncArray<kernel_type> &diag() const;
    size_t n_instances() const { return n_instances_; }
    size_t n_features() const { return n_features_; }
    size_t nnz() const { return nnz_; }
    tsvm_km *handle() const { return km_; }
    bool stored_dense() const { return dense_; }
    const SvmParam &get_param() const { return param_; }

private:
    size_t n_instances_ = 0, n_features_ = 0, nnz_ = 0;
    bool dense_ = false;
    SvmParam param_;
    tsvm_km *km_ = nullptr;
    float *pair_x_ = nullptr;          // device copy of the two row blocks (second constructor)
    mutable SyncArray<kernel_type> diag_;
};
#endif
