// Prediction: decision values of a batch of test instances against the support vectors.
// Reference behaviour: SvmModel::predict_dec_values (src/thundersvm/model/svmmodel.cpp:74-117),
// svm_kernel::sum_kernel_values (src/thundersvm/kernel/kernelmatrix_kernel.cu:69-97) and the
// vote of SVC::predict_label (src/thundersvm/model/svc.cpp:265-289).
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

extern "C" {

tsvm_status tsvm_predict_dec(tsvm_km *km_sv, const double *coef_dev, const int *sv_count_host, const double *rho_dev,
                             int n_classes, int m, const float *T_dev, int dt, int ldt, const float *tval_dev,
                             const int *trow_ptr_dev, const int *tcol_dev, long long tnnz, double *dec_dev,
                             size_t max_mem_bytes, void *stream) {
    TSVM_REQUIRE(km_sv && coef_dev && sv_count_host && rho_dev && dec_dev && n_classes >= 2 && m > 0,
                 "predict_dec: bad arguments");
    TSVM_REQUIRE(T_dev || trow_ptr_dev, "predict_dec: neither a dense nor a CSR test batch was given");
    cudaStream_t st = (cudaStream_t) stream;
    const int n_sv = km_sv->n;
    int total = 0;
    std::vector<int> start(n_classes), count(n_classes);
    for (int c = 0; c < n_classes; ++c) { start[c] = total; count[c] = sv_count_host[c]; total += count[c]; }
    TSVM_REQUIRE(total == n_sv, "predict_dec: support-vector counts sum to %d but the matrix holds %d", total, n_sv);
    // batch rows so that the kernel-value buffer stays within the budget (svmmodel.cpp:86-89 caps at 10000)
    const long long ldk = ((long long) n_sv + 3) & ~3ll;
    size_t budget = max_mem_bytes;
    if (!budget) {                 // no cap given: a quarter of what is free (the reference batches by its own cap)
        size_t free_b = 0, total_b = 0;
        budget = cudaMemGetInfo(&free_b, &total_b) == cudaSuccess ? free_b / 4 : ((size_t) 2 << 30);
        if (budget < ((size_t) 256 << 20)) budget = (size_t) 256 << 20;
    }
    long long batch = (long long) (budget / sizeof(float) / (size_t) ldk);
    if (batch > 10000) batch = 10000;
    if (batch > m) batch = m;
    if (batch < 1) batch = 1;
    float *K = nullptr;
    int *meta = nullptr;
    TSVM_TRY(dev_alloc(&K, (size_t) batch * ldk));
    tsvm_status s = dev_alloc(&meta, (size_t) 2 * n_classes);
    if (s == TSVM_OK) {
        cudaError_t e = cudaMemcpyAsync(meta, start.data(), sizeof(int) * n_classes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(meta + n_classes, count.data(), sizeof(int) * n_classes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);   // start/count are stack-local
        if (e != cudaSuccess) { set_error("predict_dec: metadata copy failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
    }
    const int nb = n_classes * (n_classes - 1) / 2;
    for (long long r0 = 0; r0 < m && s == TSVM_OK; r0 += batch) {
        const int mm = (int) ((m - r0) < batch ? (m - r0) : batch);
        if (T_dev) s = tsvm_km_rows_by_instances_dense(km_sv, T_dev + (size_t) r0 * ldt, mm, dt, ldt, K, ldk, st);
        else s = tsvm_km_rows_by_instances_csr(km_sv, tval_dev, trow_ptr_dev + r0, tcol_dev, mm, tnnz, K, ldk, st);
        if (s != TSVM_OK) break;
        sum_kernel_values_kernel<<<mm, 256, 0, st>>>(coef_dev, n_sv, meta, meta + n_classes, rho_dev, K, ldk,
                                                     dec_dev + (size_t) r0 * nb, n_classes);
        count_launch();
        if (cudaPeekAtLastError() != cudaSuccess) { set_error("sum_kernel_values launch failed"); s = TSVM_ERR_CUDA; }
    }
    if (s == TSVM_OK) {
        cudaError_t e = cudaMemcpyAsync(km_sv->status_host, km_sv->status_dev, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) { set_error("predict_dec failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
        else if (km_sv->status_host[0] != 0) {
            set_error("dense kernel-row engine reported status %d (a bounded wait ran out)", km_sv->status_host[0]);
            s = TSVM_ERR_DEVICE;
        }
    } else cudaStreamSynchronize(st);
    pool_free_many({K, meta});
    return s;
}

tsvm_status tsvm_vote(const double *dec_dev, int m, int n_classes, int *out_dev, void *stream) {
    TSVM_REQUIRE(dec_dev && out_dev && m > 0 && n_classes >= 2, "vote: bad arguments");
    TSVM_LAUNCH(vote_kernel, ceil_div(m, 128), 128, 0, (cudaStream_t) stream, dec_dev, m, n_classes, out_dev);
    return TSVM_OK;
}

}  // extern "C"
