// Shared helpers for the sm_100a kernels: status/error plumbing, launch accounting,
// order-preserving keys and warp reductions.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <math.h>
#include <atomic>
#include <initializer_list>
#include "../../include/thundersvm_b200.h"

namespace tsvm {

void set_error(const char *fmt, ...);
long long launch_count();
void count_launch(int k = 1);

#define TSVM_CUDA(expr)                                                                          \
    do {                                                                                         \
        cudaError_t e__ = (expr);                                                                \
        if (e__ != cudaSuccess) {                                                                \
            tsvm::set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__,                 \
                            cudaGetErrorString(e__));                                            \
            return e__ == cudaErrorMemoryAllocation ? TSVM_ERR_OOM : TSVM_ERR_CUDA;              \
        }                                                                                        \
    } while (0)

#define TSVM_TRY(expr)                        \
    do {                                      \
        tsvm_status s__ = (expr);             \
        if (s__ != TSVM_OK) return s__;       \
    } while (0)

#define TSVM_REQUIRE(cond, ...)               \
    do {                                      \
        if (!(cond)) {                        \
            tsvm::set_error(__VA_ARGS__);     \
            return TSVM_ERR_INVALID;          \
        }                                     \
    } while (0)

// Launch + account + check the launch (not the execution).
#define TSVM_LAUNCH(kernel, grid, block, smem, stream, ...)                                      \
    do {                                                                                         \
        kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);                              \
        tsvm::count_launch();                                                                    \
        TSVM_CUDA(cudaPeekAtLastError());                                                        \
    } while (0)

// One-time set-up that belongs to a device, not to the process (cudaFuncSetAttribute applies to the device
// that is current when it runs): the statement runs on the first use on every device ordinal. Two threads
// that meet here for the same device both run it; the set-ups are idempotent, so that race is harmless.
constexpr int MAX_DEVICES = 64;
#define TSVM_ONCE_PER_DEVICE(...)                                                                \
    do {                                                                                         \
        static std::atomic<unsigned long long> done__{0};                                        \
        int dev__ = 0;                                                                           \
        TSVM_CUDA(cudaGetDevice(&dev__));                                                        \
        const unsigned long long bit__ = 1ull << (dev__ & (tsvm::MAX_DEVICES - 1));              \
        if (!(done__.load(std::memory_order_acquire) & bit__)) {                                 \
            __VA_ARGS__;                                                                         \
            done__.fetch_or(bit__, std::memory_order_release);                                   \
        }                                                                                        \
    } while (0)

// Device and pinned-host memory of the handles comes from a per-process pool (km.cu): a freed block is
// kept and handed out again for a request of the same size class instead of going back to the driver.
// Training a multi-class model creates and destroys a kernel matrix and a solver per class pair; the
// driver's allocation calls cost more than such a sub-problem's whole solve.
tsvm_status pool_alloc(void **p, size_t bytes);
void pool_free(void *p);                      // waits for the block's device, like cudaFree
// Several blocks at once: one wait per device that owns any of them, then all are filed.
void pool_free_many(std::initializer_list<void *> blocks);
void pool_release();                          // returns every cached block to the driver
tsvm_status pinned_alloc(void **p, size_t bytes);
void pinned_free(void *p);

template <typename T>
inline tsvm_status dev_alloc(T **p, size_t count) {
    *p = nullptr;
    if (count == 0) count = 1;
    return pool_alloc((void **) p, count * sizeof(T));
}

inline int ceil_div(long long a, long long b) { return (int) ((a + b - 1) / b); }

// ---- device helpers ------------------------------------------------------------------

// Monotone map double -> uint64 (ascending); -0.0 is folded onto +0.0 so that equal values
// get equal keys.
__host__ __device__ __forceinline__ unsigned long long ordered_key(double v) {
    if (v == 0.0) v = 0.0;
#ifdef __CUDA_ARCH__
    unsigned long long b = (unsigned long long) __double_as_longlong(v);
#else
    unsigned long long b;
    memcpy(&b, &v, 8);
#endif
    return (b & 0x8000000000000000ull) ? ~b : (b | 0x8000000000000000ull);
}

__host__ __device__ __forceinline__ double key_to_double(unsigned long long k) {
    unsigned long long b = (k & 0x8000000000000000ull) ? (k & 0x7fffffffffffffffull) : ~k;
#ifdef __CUDA_ARCH__
    return __longlong_as_double((long long) b);
#else
    double v;
    memcpy(&v, &b, 8);
    return v;
#endif
}

// I_up / I_low / free membership, include/thundersvm/kernel/smo_kernel.h:13-23
__host__ __device__ __forceinline__ bool in_I_up(double a, int y, double Cp, double Cn) {
    return (y > 0 && a < Cp) || (y < 0 && a > 0);
}
__host__ __device__ __forceinline__ bool in_I_low(double a, int y, double Cp, double Cn) {
    return (y > 0 && a > 0) || (y < 0 && a < Cn);
}
__host__ __device__ __forceinline__ bool is_free_sv(double a, int y, double Cp, double Cn) {
    return a > 0 && (y > 0 ? a < Cp : a < Cn);
}

#ifdef __CUDACC__
// Warp-wide minimum of a 64-bit key and the lowest `slot` among the lanes that hold it.
__device__ __forceinline__ void warp_argmin_u64(unsigned long long &key, int &slot) {
    const unsigned full = 0xffffffffu;
    unsigned hi = (unsigned) (key >> 32), lo = (unsigned) key;
    unsigned mhi = __reduce_min_sync(full, hi);
    unsigned mlo = __reduce_min_sync(full, hi == mhi ? lo : 0xffffffffu);
    bool win = (hi == mhi) && (lo == mlo);
    unsigned ms = __reduce_min_sync(full, win ? (unsigned) slot : 0x7fffffffu);
    key = ((unsigned long long) mhi << 32) | mlo;
    slot = (int) ms;
}

__device__ __forceinline__ unsigned long long warp_min_u64(unsigned long long key) {
    const unsigned full = 0xffffffffu;
    unsigned hi = (unsigned) (key >> 32), lo = (unsigned) key;
    unsigned mhi = __reduce_min_sync(full, hi);
    unsigned mlo = __reduce_min_sync(full, hi == mhi ? lo : 0xffffffffu);
    return ((unsigned long long) mhi << 32) | mlo;
}
#endif

// The reference's kernel functions (src/thundersvm/kernel/kernelmatrix_kernel.cu:47-67,
// 141-152): RBF expf(-(sd_i + sd_j - 2 dot) gamma), poly powf(gamma dot + coef0, degree),
// sigmoid tanhf(gamma dot + coef0), linear = dot.
struct KernelFn {
    int type;
    int degree;
    float gamma;
    float coef0;
};

__device__ __forceinline__ float apply_kernel(const KernelFn &k, float dot, float sd_i, float sd_j) {
    switch (k.type) {
        case TSVM_RBF:
        case TSVM_PRECOMPUTED:
            return expf(-(sd_i + sd_j - dot * 2.0f) * k.gamma);
        case TSVM_POLY:
            return powf(k.gamma * dot + k.coef0, (float) k.degree);
        case TSVM_SIGMOID:
            return tanhf(k.gamma * dot + k.coef0);
        default:
            return dot;
    }
}

}  // namespace tsvm

// A set of instances as the tensor engines read it: two operand planes (row stride = the handle's plane_ld),
// self dots and, for FP16 planes, 1/scale of every row.
struct InstancePlanes {
    const float *hi, *lo, *sd, *unscale;
    int n;
};
// The requested rows in the same form (nullptr hi: the handle's own staging buffers).
struct RowPlanes {
    const float *hi, *lo, *sd, *unscale;
};

// Opaque handle behind tsvm_km.
struct tsvm_km {
    int n = 0, d = 0;
    long long nnz = 0;
    bool dense = true;
    tsvm::KernelFn fn{};
    // 0 = automatic, 1 = CUDA-core FP32, 2 = tcgen05 TF32 planes single CTA, 3 = tcgen05 TF32 planes CTA pairs,
    // 4 = tcgen05 row-scaled FP16 planes CTA pairs
    int engine = 0;
    // dense storage: row-major, row stride ldx floats (multiple of 4)
    const float *X = nullptr;
    int ldx = 0;
    float *X_owned = nullptr;
    // Two-plane split of X for the tensor engines, built on first use: TF32 words (plane_kind 1, row
    // stride d_pad) or row-scaled FP16 halves (plane_kind 2, row stride plane_ld = round_up(d, 8)).
    float *Xhi = nullptr, *Xlo = nullptr;
    int plane_kind = 0, plane_ld = 0;
    float *x_unscale = nullptr;     // FP16 planes: 1 / (power-of-two scale) of every instance row [n]
    int d_pad = 0;
    // CSR storage
    const float *val = nullptr;
    const int *row_ptr = nullptr, *col = nullptr;
    float *val_owned = nullptr;
    int *row_ptr_owned = nullptr, *col_owned = nullptr;
    float *self_dot = nullptr, *diag = nullptr;
    // scratch for the rows whose kernel values are requested
    int w_cap = 0;                  // rows the scratch below can hold
    float *W = nullptr;             // dense engines: w_cap x d_pad (row-major), FP32
    float *Whi = nullptr, *Wlo = nullptr;   // two-plane split of W, same kind as the X planes
    float *w_unscale = nullptr;     // FP16 planes: 1 / scale of every requested row [w_cap]
    float *WT = nullptr;            // CSR engine: d x wt_ld, column = requested row
    int wt_ld = 0;
    float *sd_rows = nullptr;       // self dots of the requested rows [w_cap]
    int reserve_clusters = 0;       // SM pairs the pair engine leaves free (a concurrent stream's kernels run there)
    // Set by a caller around tsvm_km_rows_by_index-style launches (the solver's row cache): the number of
    // requested rows is read from the device (at most the q of the call) and requested row i goes to row
    // rows_slot_dev[i] of the output buffer instead of row i.
    const int *rows_m_dev = nullptr, *rows_slot_dev = nullptr;
    int *status_dev = nullptr;      // device status word written by kernels with bounded waits
    int *status_host = nullptr;     // pinned mirror
};

namespace tsvm {
// Pieces of tsvm_km_rows_by_index (km.cu) for callers that overlap them with other work.
bool km_pair_engine(tsvm_km *km, cudaStream_t st);
size_t km_plane_row_bytes(const tsvm_km *km);
tsvm_status km_stage_rows_by_index(tsvm_km *km, const int *idx_dev, int q, cudaStream_t st);
tsvm_status km_rows_staged(tsvm_km *km, int q, float *out, long long ld_out, cudaStream_t st);
// operand planes of instances ids[0..m) (m_dev: only the first *m_dev of them, read on the device)
tsvm_status km_gather_planes(tsvm_km *km, const int *ids_dev, int m, const int *m_dev, float *hi, float *lo, float *sd,
                             float *unscale, cudaStream_t st);
tsvm_status km_rows_staged_on(tsvm_km *km, const InstancePlanes &X, int q, float *out, long long ld_out,
                              cudaStream_t st);
tsvm_status km_rows_planes_on(tsvm_km *km, const InstancePlanes &X, const RowPlanes &W, int q, float *out,
                              long long ld_out, cudaStream_t st);
tsvm_status km_stage_instances_dense(tsvm_km *km, const float *T, int mm, int dt, int ldt, cudaStream_t st);
tsvm_status km_stage_instances_csr(tsvm_km *km, const float *tval, const int *rp, const int *tcol, int mm,
                                   cudaStream_t st);
tsvm_status launch_dense_tc2_predict(tsvm_km *km, int m, const double *coef_dev, const int *sv_class_dev,
                                     int n_classes, double *dec_dev, cudaStream_t st);
tsvm_status km_stage_rows_features(tsvm_km *km, const float *T_dev, int ldt, const float *sd_T_dev, int m,
                                   cudaStream_t st);
}  // namespace tsvm
