// Prediction: decision values of a batch of test instances against the support vectors.
// Reference behaviour: SvmModel::predict_dec_values (src/thundersvm/model/svmmodel.cpp:74-117),
// svm_kernel::sum_kernel_values (src/thundersvm/kernel/kernelmatrix_kernel.cu:69-97), the vote of
// SVC::predict_label (src/thundersvm/model/svc.cpp:265-289) and the vote-only form
// sum_kernel_values_instant (kernelmatrix_kernel.cu:99-138).
//
// Dense support vectors on the CTA-pair tensor engine take the fused path: the test x SV contraction
// multiplies its kernel values by the coefficients in its epilogue and adds them to the decision values
// (dense_tc2.cu, prediction form), so the kernel block is never written. Other storages (CSR support
// vectors, at most 32 features) compute the block in slabs of test rows and reduce it with
// sum_kernel_values_kernel.
#include "common.cuh"
#include <vector>

namespace tsvm {

// One block per test row. For every class pair (i, j), i < j, in the reference's order:
//   dec = sum_{s in class i} coef[(j-1) n_sv + s] K[s] + sum_{s in class j} coef[i n_sv + s] K[s] - rho[k]
// with double accumulation; K and coef are read with unit stride across the block.
__global__ void __launch_bounds__(256)
sum_kernel_values_kernel(const double *__restrict__ coef, int n_sv, const int *__restrict__ sv_start,
                         const int *__restrict__ sv_count, const double *__restrict__ rho,
                         const float *__restrict__ K, long long ldk, double *__restrict__ dec, int n_classes) {
    __shared__ double part[2][8];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *kv = K + (size_t) r * ldk;
    const int nb = n_classes * (n_classes - 1) / 2;
    int k = 0;
    for (int i = 0; i < n_classes; ++i)
        for (int j = i + 1; j < n_classes; ++j, ++k) {
            const double *c1 = coef + (size_t) (j - 1) * n_sv + sv_start[i];
            const double *c2 = coef + (size_t) i * n_sv + sv_start[j];
            const float *k1 = kv + sv_start[i], *k2 = kv + sv_start[j];
            const int n1 = sv_count[i], n2 = sv_count[j];
            double s = 0;
            for (int l = tid; l < n1; l += 256) s += c1[l] * (double) k1[l];
            for (int l = tid; l < n2; l += 256) s += c2[l] * (double) k2[l];
            for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            double *buf = part[k & 1];
            if (lane == 0) buf[warp] = s;
            __syncthreads();
            if (tid == 0) {
                double t = 0;
                for (int w = 0; w < 8; ++w) t += buf[w];
                dec[(size_t) r * nb + k] = t - rho[k];
            }
        }
}

// dec[r][k] = -rho[k]: the fused contraction then adds its sums
__global__ void preset_dec_kernel(double *__restrict__ dec, long long total, int nb, const double *__restrict__ rho) {
    const long long e = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (e < total) dec[e] = -rho[e % nb];
}

// class of every support vector from the per-class start offsets
__global__ void sv_class_kernel(int *__restrict__ cls, int n_sv, const int *__restrict__ sv_start, int n_classes) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_sv) return;
    int c = 0;
    while (c + 1 < n_classes && s >= sv_start[c + 1]) ++c;
    cls[s] = c;
}

// votes -> index of the winning class, first maximum wins
__global__ void vote_kernel(const double *__restrict__ dec, int m, int n_classes, int *__restrict__ out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= m) return;
    const int nb = n_classes * (n_classes - 1) / 2;
    int best = 0, best_votes = -1;
    for (int c = 0; c < n_classes; ++c) {
        int votes = 0, k = 0;
        for (int i = 0; i < n_classes; ++i)
            for (int j = i + 1; j < n_classes; ++j, ++k) {
                const bool pos = dec[(size_t) r * nb + k] > 0;
                if ((pos && i == c) || (!pos && j == c)) ++votes;
            }
        if (votes > best_votes) { best_votes = votes; best = c; }
    }
    out[r] = best;
}

}  // namespace tsvm

using namespace tsvm;

// Rows of test instances handled per launch of the fused contraction (the handle's staging scratch grows
// to hold them) and per slab of the unfused path.
static constexpr int FUSED_ROWS = 4096;

// Decision values of test rows [r0, r0 + mm) into dec (mm x nb, preset here), fused path.
static tsvm_status fused_slab(tsvm_km *km_sv, const double *coef_dev, const int *sv_class, const double *rho_dev,
                              int n_classes, long long r0, int mm, const float *T_dev, int dt, int ldt,
                              const float *tval_dev, const int *trow_ptr_dev, const int *tcol_dev, double *dec,
                              cudaStream_t st) {
    const int nb = n_classes * (n_classes - 1) / 2;
    const long long total = (long long) mm * nb;
    TSVM_LAUNCH(preset_dec_kernel, ceil_div(total, 256), 256, 0, st, dec, total, nb, rho_dev);
    if (T_dev) TSVM_TRY(km_stage_instances_dense(km_sv, T_dev + (size_t) r0 * ldt, mm, dt, ldt, st));
    else TSVM_TRY(km_stage_instances_csr(km_sv, tval_dev, trow_ptr_dev + r0, tcol_dev, mm, st));
    return launch_dense_tc2_predict(km_sv, mm, coef_dev, sv_class, n_classes, dec, st);
}

// labels_dev != nullptr: only the vote leaves the slab (sum_kernel_values_instant); dec_dev is then unused.
static tsvm_status predict_impl(tsvm_km *km_sv, const double *coef_dev, const int *sv_count_host, const double *rho_dev,
                                int n_classes, int m, const float *T_dev, int dt, int ldt, const float *tval_dev,
                                const int *trow_ptr_dev, const int *tcol_dev, double *dec_dev, int *labels_dev,
                                size_t max_mem_bytes, cudaStream_t st) {
    const int n_sv = km_sv->n;
    int total = 0;
    std::vector<int> start(n_classes), count(n_classes);
    for (int c = 0; c < n_classes; ++c) { start[c] = total; count[c] = sv_count_host[c]; total += count[c]; }
    TSVM_REQUIRE(total == n_sv, "predict: support-vector counts sum to %d but the matrix holds %d", total, n_sv);
    const int nb = n_classes * (n_classes - 1) / 2;
    const bool fused = km_pair_engine(km_sv, st);
    const long long ldk = ((long long) n_sv + 3) & ~3ll;
    long long batch = FUSED_ROWS;
    if (!fused) {
        // the kernel block of a slab must fit the budget (svmmodel.cpp:86-89 caps a batch at 10000 rows)
        size_t budget = max_mem_bytes;
        if (!budget) {
            size_t free_b = 0, total_b = 0;
            budget = cudaMemGetInfo(&free_b, &total_b) == cudaSuccess ? free_b / 4 : ((size_t) 2 << 30);
            if (budget < ((size_t) 256 << 20)) budget = (size_t) 256 << 20;
        }
        batch = (long long) (budget / sizeof(float) / (size_t) ldk);
        if (batch > 10000) batch = 10000;
    }
    if (batch > m) batch = m;
    if (batch < 1) batch = 1;
    float *K = nullptr;
    int *meta = nullptr, *sv_class = nullptr;
    double *dec_slab = nullptr;
    tsvm_status s = dev_alloc(&meta, (size_t) 2 * n_classes);
    if (s == TSVM_OK && !fused) s = dev_alloc(&K, (size_t) batch * ldk);
    if (s == TSVM_OK && fused) s = dev_alloc(&sv_class, (size_t) n_sv);
    if (s == TSVM_OK && labels_dev) s = dev_alloc(&dec_slab, (size_t) batch * nb);
    if (s == TSVM_OK) {
        cudaError_t e = cudaMemcpyAsync(meta, start.data(), sizeof(int) * n_classes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(meta + n_classes, count.data(), sizeof(int) * n_classes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);   // start/count are stack-local
        if (e != cudaSuccess) { set_error("predict: metadata copy failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
    }
    auto run = [&]() -> tsvm_status {
        if (fused) TSVM_LAUNCH(sv_class_kernel, ceil_div(n_sv, 256), 256, 0, st, sv_class, n_sv, meta, n_classes);
        for (long long r0 = 0; r0 < m; r0 += batch) {
            const int mm = (int) ((m - r0) < batch ? (m - r0) : batch);
            double *dec = labels_dev ? dec_slab : dec_dev + (size_t) r0 * nb;
            if (fused) {
                TSVM_TRY(fused_slab(km_sv, coef_dev, sv_class, rho_dev, n_classes, r0, mm, T_dev, dt, ldt, tval_dev,
                                    trow_ptr_dev, tcol_dev, dec, st));
            } else {
                if (T_dev) TSVM_TRY(tsvm_km_rows_by_instances_dense(km_sv, T_dev + (size_t) r0 * ldt, mm, dt, ldt, K, ldk, st));
                else TSVM_TRY(tsvm_km_rows_by_instances_csr(km_sv, tval_dev, trow_ptr_dev + r0, tcol_dev, mm, 0, K, ldk, st));
                TSVM_LAUNCH(sum_kernel_values_kernel, mm, 256, 0, st, coef_dev, n_sv, meta, meta + n_classes, rho_dev, K,
                            ldk, dec, n_classes);
            }
            if (labels_dev)
                TSVM_LAUNCH(vote_kernel, ceil_div(mm, 128), 128, 0, st, dec, mm, n_classes, labels_dev + r0);
        }
        return TSVM_OK;
    };
    if (s == TSVM_OK) s = run();
    if (s == TSVM_OK) {
        cudaError_t e = cudaMemcpyAsync(km_sv->status_host, km_sv->status_dev, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) { set_error("predict failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
        else if (km_sv->status_host[0] != 0) {
            set_error("dense kernel-row engine reported status %d (a bounded wait ran out)", km_sv->status_host[0]);
            s = TSVM_ERR_DEVICE;
        }
    } else cudaStreamSynchronize(st);
    pool_free_many({K, meta, sv_class, dec_slab});
    return s;
}

extern "C" {

tsvm_status tsvm_predict_dec(tsvm_km *km_sv, const double *coef_dev, const int *sv_count_host, const double *rho_dev,
                             int n_classes, int m, const float *T_dev, int dt, int ldt, const float *tval_dev,
                             const int *trow_ptr_dev, const int *tcol_dev, long long tnnz, double *dec_dev,
                             size_t max_mem_bytes, void *stream) {
    (void) tnnz;
    TSVM_REQUIRE(km_sv && coef_dev && sv_count_host && rho_dev && dec_dev && n_classes >= 2 && m > 0,
                 "predict_dec: bad arguments");
    TSVM_REQUIRE(T_dev || trow_ptr_dev, "predict_dec: neither a dense nor a CSR test batch was given");
    return predict_impl(km_sv, coef_dev, sv_count_host, rho_dev, n_classes, m, T_dev, dt, ldt, tval_dev, trow_ptr_dev,
                        tcol_dev, dec_dev, nullptr, max_mem_bytes, (cudaStream_t) stream);
}

tsvm_status tsvm_predict_labels(tsvm_km *km_sv, const double *coef_dev, const int *sv_count_host,
                                const double *rho_dev, int n_classes, int m, const float *T_dev, int dt, int ldt,
                                const float *tval_dev, const int *trow_ptr_dev, const int *tcol_dev, long long tnnz,
                                int *labels_dev, size_t max_mem_bytes, void *stream) {
    (void) tnnz;
    TSVM_REQUIRE(km_sv && coef_dev && sv_count_host && rho_dev && labels_dev && n_classes >= 2 && m > 0,
                 "predict_labels: bad arguments");
    TSVM_REQUIRE(T_dev || trow_ptr_dev, "predict_labels: neither a dense nor a CSR test batch was given");
    return predict_impl(km_sv, coef_dev, sv_count_host, rho_dev, n_classes, m, T_dev, dt, ldt, tval_dev, trow_ptr_dev,
                        tcol_dev, nullptr, labels_dev, max_mem_bytes, (cudaStream_t) stream);
}

tsvm_status tsvm_vote(const double *dec_dev, int m, int n_classes, int *out_dev, void *stream) {
    TSVM_REQUIRE(dec_dev && out_dev && m > 0 && n_classes >= 2, "vote: bad arguments");
    TSVM_LAUNCH(vote_kernel, ceil_div(m, 128), 128, 0, (cudaStream_t) stream, dec_dev, m, n_classes, out_dev);
    return TSVM_OK;
}

}  // extern "C"
