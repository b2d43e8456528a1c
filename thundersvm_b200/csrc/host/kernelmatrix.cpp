// KernelMatrix, CSMOSolver and NuSMOSolver: thin forwards to the C ABI (include/thundersvm_b200.h).
// Reference behaviour: src/thundersvm/kernelmatrix.cpp:183-316, src/thundersvm/solver/csmosolver.cpp:10-121.
#include <thundersvm/kernelmatrix.h>
#include <thundersvm/solver/csmosolver.h>
#include <thundersvm/solver/nusmosolver.h>
#include <cuda_runtime.h>
#include "../../../include/thundersvm_b200.h"

namespace {
void b200_check(tsvm_status s) {
    if (s == TSVM_OK) return;
    if (s == TSVM_ERR_OOM) throw std::bad_alloc();
    LOG(FATAL) << "thundersvm_b200: " << tsvm_last_error();
}

// node2d -> CSR with the ids as they are (1-based from LibSVM text); returns max id + 1
struct HostCsr {
    vector<float> val;
    vector<int> col, row_ptr;
    int n_features = 0;
};
HostCsr to_csr(const DataSet::node2d &ins) {
    HostCsr c;
    size_t nnz = 0;
    for (auto &r : ins) nnz += r.size();
    c.val.reserve(nnz); c.col.reserve(nnz); c.row_ptr.reserve(ins.size() + 1);
    c.row_ptr.push_back(0);
    int mx = 0;
    for (auto &r : ins) {
        for (auto &nd : r) {
            c.val.push_back(nd.value);
            c.col.push_back(nd.index);
            if (nd.index > mx) mx = nd.index;
        }
        c.row_ptr.push_back((int) c.val.size());
    }
    c.n_features = mx + 1;            // column 0 stays empty for one-based data (kernelmatrix.cpp:200-206)
    return c;
}
}  // namespace

KernelMatrix::KernelMatrix(const DataSet::node2d &instances, SvmParam param) : param_(param) {
    n_instances_ = instances.size();
    CHECK(n_instances_ > 0) << "KernelMatrix needs at least one instance";
    HostCsr c = to_csr(instances);
    n_features_ = c.n_features;
    nnz_ = c.val.size();
    // Storage: the tensor-core engine wants a dense row-major matrix; it pays off unless the data
    // is very sparse (then the CSR engine touches far fewer bytes) or the three dense planes would
    // not fit next to the kernel-row buffer.
    const double density = (double) nnz_ / ((double) n_instances_ * n_features_);
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    const double dense_bytes = 3.0 * n_instances_ * ((n_features_ + 3) & ~3ul) * 4.0 + 1024.0 * n_instances_ * 4.0;
    dense_ = (density >= 0.02 || n_features_ <= 256) && dense_bytes < 0.6 * (double) free_b;
    if (dense_) {
        vector<float> X(n_instances_ * n_features_, 0.0f);
#pragma omp parallel for schedule(static)
        for (long i = 0; i < (long) n_instances_; ++i)
            for (int p = c.row_ptr[i]; p < c.row_ptr[i + 1]; ++p) X[(size_t) i * n_features_ + c.col[p]] = c.val[p];
        b200_check(tsvm_km_create_dense(X.data(), (int) n_instances_, (int) n_features_, (int) n_features_, TSVM_HOST,
                                        param.kernel_type, param.degree, (float) param.gamma, (float) param.coef0,
                                        thundersvm::work_stream(), &km_));
    } else {
        b200_check(tsvm_km_create_csr(c.val.data(), c.row_ptr.data(), c.col.data(), (int) n_instances_,
                                      (int) n_features_, TSVM_HOST, param.kernel_type, param.degree,
                                      (float) param.gamma, (float) param.coef0, thundersvm::work_stream(), &km_));
    }
    cudaStreamSynchronize(thundersvm::work_stream());    // the host staging buffers above go out of scope
    thundersvm::total_memory_size() += (dense_ ? (size_t) dense_bytes : nnz_ * 8 + n_instances_ * 12);
    diag_.resize(n_instances_);
    thundersvm::copy_to_host(diag_.host_data(), tsvm_km_diag_dev(km_), sizeof(kernel_type) * n_instances_);
}

KernelMatrix::KernelMatrix(const float *X_dev, size_t d, size_t ld, size_t r0, size_t n0, size_t r1, size_t n1,
                           SvmParam param) : param_(param) {
    n_instances_ = n0 + n1;
    n_features_ = d;
    nnz_ = n_instances_ * d;
    dense_ = true;
    CHECK(n_instances_ > 0) << "KernelMatrix needs at least one instance";
    pair_x_ = static_cast<float *>(thundersvm::device_alloc(n_instances_ * ld * sizeof(float)));
    thundersvm::copy_on_device(pair_x_, X_dev + r0 * ld, n0 * ld * sizeof(float));
    thundersvm::copy_on_device(pair_x_ + n0 * ld, X_dev + r1 * ld, n1 * ld * sizeof(float));
    b200_check(tsvm_km_create_dense(pair_x_, (int) n_instances_, (int) d, (int) ld, TSVM_DEVICE, param.kernel_type,
                                    param.degree, (float) param.gamma, (float) param.coef0, thundersvm::work_stream(), &km_));
    const double dense_bytes = 3.0 * n_instances_ * ((n_features_ + 3) & ~3ul) * 4.0 + 1024.0 * n_instances_ * 4.0;
    thundersvm::total_memory_size() += (size_t) dense_bytes;
    diag_.resize(n_instances_);
    thundersvm::copy_to_host(diag_.host_data(), tsvm_km_diag_dev(km_), sizeof(kernel_type) * n_instances_);
}

KernelMatrix::~KernelMatrix() {
    if (km_) {
        const double dense_bytes = 3.0 * n_instances_ * ((n_features_ + 3) & ~3ul) * 4.0 + 1024.0 * n_instances_ * 4.0;
        thundersvm::total_memory_size() -= (dense_ ? (size_t) dense_bytes : nnz_ * 8 + n_instances_ * 12);
        tsvm_km_destroy(km_);
    }
    thundersvm::device_free(pair_x_);
}

void KernelMatrix::get_rows(const SyncArray<int> &idx, SyncArray<kernel_type> &kernel_rows) const {
    CHECK_GE(kernel_rows.size(), idx.size() * n_instances_) << "kernel_rows memory is too small";
    b200_check(tsvm_km_rows_by_index(km_, idx.device_data(), (int) idx.size(), kernel_rows.device_data(),
                                     (long long) n_instances_, thundersvm::work_stream()));
}

void KernelMatrix::get_rows(const DataSet::node2d &instances, SyncArray<kernel_type> &kernel_rows) const {
    CHECK_GE(kernel_rows.size(), instances.size() * n_instances_) << "kernel_rows memory is too small";
    if (instances.empty()) return;
    HostCsr c = to_csr(instances);
    SyncArray<kernel_type> val(std::max<size_t>(c.val.size(), 1));
    SyncArray<int> col(std::max<size_t>(c.col.size(), 1)), rp(c.row_ptr.size());
    if (!c.val.empty()) { val.copy_from(c.val.data(), c.val.size()); col.copy_from(c.col.data(), c.col.size()); }
    rp.copy_from(c.row_ptr.data(), c.row_ptr.size());
    b200_check(tsvm_km_rows_by_instances_csr(km_, val.device_data(), rp.device_data(), col.device_data(),
                                             (int) instances.size(), (long long) c.val.size(), kernel_rows.device_data(),
                                             (long long) n_instances_, thundersvm::work_stream()));
    cudaStreamSynchronize(thundersvm::work_stream());
}

const SyncArray<kernel_type> &KernelMatrix::diag() const { return diag_; }

int CSMOSolver::solver_kind() const { return TSVM_SOLVER_C; }
int NuSMOSolver::solver_kind() const { return for_svr ? TSVM_SOLVER_NU_SVR : TSVM_SOLVER_NU_SVC; }

void CSMOSolver::solve(const KernelMatrix &k_mat, const SyncArray<int> &y, SyncArray<float_type> &alpha,
                       float_type &rho, SyncArray<float_type> &f_val, float_type eps, float_type Cp, float_type Cn,
                       int ws_size, int max_iter) const {
    LOG(INFO) << "training start";
    tsvm_solve_stats st;
    double rho_out = 0;
    b200_check(tsvm_smo_solve(k_mat.handle(), solver_kind(), y.device_data(), alpha.device_data(), f_val.device_data(),
                              eps, Cp, Cn, ws_size, max_iter, &rho_out, &st, thundersvm::work_stream()));
    rho = rho_out;
    LOG(INFO) << "global iter = " << st.outer_iters - 1 << ", total local iter = " << st.local_iters << ", diff = "
              << st.final_diff;
    LOG(INFO) << "training finished";
    LOG(INFO) << "obj = " << st.objective;
}
