// KernelMatrix on the device: construction, self dots / diagonal, and kernel rows for the
// CSR engine and the CUDA-core dense engine. The tensor-core dense engine lives in
// dense_tc.cu. Reference behaviour: src/thundersvm/kernelmatrix.cpp:183-316,385-406.
#include "common.cuh"
#include <cuda_fp16.h>
#include <string.h>
#include <stdlib.h>
#include <atomic>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace tsvm {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
long long launch_count() { return g_launches.load(); }
void count_launch(int k) { g_launches.fetch_add(k); }

// ---- memory pool -------------------------------------------------------------------------------------
// Size classes: eight per power of two (at most 12.5 % slack), 512 bytes at least. Blocks are per device.
namespace {
struct PoolBlock { int dev; size_t cls; };
// never destroyed: handles may be released after the static destructors of this library have run
std::mutex &g_pool_mu = *new std::mutex;
auto &g_pool_live = *new std::unordered_map<void *, PoolBlock>;
auto &g_pinned_live = *new std::unordered_map<void *, PoolBlock>;
auto &g_pool_free = *new std::map<std::pair<int, size_t>, std::vector<void *>>;
auto &g_pinned_free = *new std::map<size_t, std::vector<void *>>;
size_t g_pool_cached = 0;               // bytes in g_pool_free

size_t size_class(size_t bytes) {
    if (bytes < 512) return 512;
    size_t p2 = 512;
    while (p2 < bytes) p2 <<= 1;          // smallest power of two >= bytes
    const size_t step = p2 >> 4;          // eighths of the previous power of two
    return (bytes + step - 1) / step * step;
}
}  // namespace

void pool_release() {
    std::lock_guard<std::mutex> lk(g_pool_mu);
    int cur = 0;
    cudaGetDevice(&cur);
    for (auto &kv : g_pool_free) {
        if (kv.second.empty()) continue;
        cudaSetDevice(kv.first.first);
        for (void *q : kv.second) cudaFree(q);
        kv.second.clear();
    }
    g_pool_cached = 0;
    cudaSetDevice(cur);
}

tsvm_status pool_alloc(void **p, size_t bytes) {
    *p = nullptr;
    int dev = 0;
    TSVM_CUDA(cudaGetDevice(&dev));
    const size_t cls = size_class(bytes);
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        auto it = g_pool_free.find({dev, cls});
        if (it != g_pool_free.end() && !it->second.empty()) {
            *p = it->second.back();
            it->second.pop_back();
            g_pool_cached -= cls;
            g_pool_live[*p] = PoolBlock{dev, cls};
            return TSVM_OK;
        }
    }
    cudaError_t e = cudaMalloc(p, cls);
    if (e == cudaErrorMemoryAllocation) {      // give the cached blocks back and try once more
        cudaGetLastError();
        pool_release();
        e = cudaMalloc(p, cls);
    }
    TSVM_CUDA(e);
    std::lock_guard<std::mutex> lk(g_pool_mu);
    g_pool_live[*p] = PoolBlock{dev, cls};
    return TSVM_OK;
}

// A freed block may be handed out again at once, so nothing in flight may still use it: one wait per device
// that owns one of the blocks (the owning device, which need not be the caller's current one), then all of
// them go to the free lists. Cached bytes above the cap go back to the driver, largest blocks first.
static size_t pool_cache_cap() {
    // TSVM_POOL_CACHE_MB, else 60 % of the current device's memory (a solver's row cache is the largest block and
    // should come back from the pool when the next solver of the same problem is created)
    static const size_t cap = [] {
        if (const char *e = getenv("TSVM_POOL_CACHE_MB")) return (size_t) strtoull(e, nullptr, 10) << 20;
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) { cudaGetLastError(); return (size_t) 32 << 30; }
        return (size_t) ((double) total_b * 0.6);
    }();
    return cap;
}

void pool_free_many(std::initializer_list<void *> blocks) {
    int cur = 0;
    bool have_cur = false;
    unsigned long long synced = 0;
    std::vector<void *> foreign;
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        for (void *p : blocks) {
            if (!p) continue;
            auto it = g_pool_live.find(p);
            if (it == g_pool_live.end()) { foreign.push_back(p); continue; }
            synced |= 1ull << (it->second.dev & (MAX_DEVICES - 1));
        }
    }
    for (int dev = 0; dev < MAX_DEVICES; ++dev) {
        if (!((synced >> dev) & 1ull)) continue;
        if (!have_cur) { cudaGetDevice(&cur); have_cur = true; }
        if (dev != cur) cudaSetDevice(dev);
        cudaDeviceSynchronize();
        if (dev != cur) cudaSetDevice(cur);
    }
    for (void *p : foreign) cudaFree(p);                     // not ours (never happens for handle memory)
    std::vector<std::pair<int, void *>> to_driver;
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        for (void *p : blocks) {
            if (!p) continue;
            auto it = g_pool_live.find(p);
            if (it == g_pool_live.end()) continue;
            g_pool_free[{it->second.dev, it->second.cls}].push_back(p);
            g_pool_cached += it->second.cls;
            g_pool_live.erase(it);
        }
        // over the cap: return the largest cached blocks first
        for (auto kv = g_pool_free.rbegin(); kv != g_pool_free.rend() && g_pool_cached > pool_cache_cap(); ++kv)
            while (!kv->second.empty() && g_pool_cached > pool_cache_cap()) {
                to_driver.push_back({kv->first.first, kv->second.back()});
                kv->second.pop_back();
                g_pool_cached -= kv->first.second;
            }
    }
    for (auto &b : to_driver) {
        if (!have_cur) { cudaGetDevice(&cur); have_cur = true; }
        if (b.first != cur) cudaSetDevice(b.first);
        cudaFree(b.second);
        if (b.first != cur) cudaSetDevice(cur);
    }
}

void pool_free(void *p) {
    if (p) pool_free_many({p});
}

tsvm_status pinned_alloc(void **p, size_t bytes) {
    *p = nullptr;
    const size_t cls = size_class(bytes);
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        auto &v = g_pinned_free[cls];
        if (!v.empty()) { *p = v.back(); v.pop_back(); g_pinned_live[*p] = PoolBlock{0, cls}; return TSVM_OK; }
    }
    TSVM_CUDA(cudaMallocHost(p, cls));
    std::lock_guard<std::mutex> lk(g_pool_mu);
    g_pinned_live[*p] = PoolBlock{0, cls};
    return TSVM_OK;
}

void pinned_free(void *p) {
    if (!p) return;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    auto it = g_pinned_live.find(p);
    if (it == g_pinned_live.end()) { cudaFreeHost(p); return; }
    g_pinned_free[it->second.cls].push_back(p);
    g_pinned_live.erase(it);
}

tsvm_status launch_dense_tc(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st);  // dense_tc.cu

// ---- construction kernels ---------------------------------------------------------------

// self_dot[i] = float(sum_k double(x_ik)^2), one warp per row (kernelmatrix.cpp:194-204).
__global__ void self_dot_dense_kernel(const float *__restrict__ X, int n, int d, int ld, float *__restrict__ out) {
    int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= n) return;
    const float *x = X + (size_t) row * ld;
    double s = 0;
    for (int k = lane; k < d; k += 32) { double v = x[k]; s += v * v; }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[row] = (float) s;
}

__global__ void self_dot_csr_kernel(const float *__restrict__ val, const int *__restrict__ row_ptr, int n,
                                    float *__restrict__ out) {
    int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= n) return;
    double s = 0;
    for (int p = row_ptr[row] + lane; p < row_ptr[row + 1]; p += 32) { double v = val[p]; s += v * v; }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[row] = (float) s;
}

// diag (kernelmatrix.cpp:225-247)
__global__ void diag_kernel(const float *__restrict__ sd, int n, KernelFn fn, float *__restrict__ out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = sd[i];
    switch (fn.type) {
        case TSVM_RBF: case TSVM_PRECOMPUTED: v = 1.0f; break;
        case TSVM_POLY: v = powf(fn.gamma * v + fn.coef0, (float) fn.degree); break;
        case TSVM_SIGMOID: v = tanhf(fn.gamma * v + fn.coef0); break;
        default: break;
    }
    out[i] = v;
}

// Self dot of a batch of new instances, accumulated sequentially in float in storage order
// as kernelmatrix.cpp:288-296 does (one thread per row keeps that order).
__global__ void self_dot_seq_dense_kernel(const float *__restrict__ T, int m, int dt, int ldt,
                                          float *__restrict__ out) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= m) return;
    const float *x = T + (size_t) r * ldt;
    float s = 0;
    for (int k = 0; k < dt; ++k) s = fmaf(x[k], x[k], s);
    out[r] = s;
}

__global__ void self_dot_seq_csr_kernel(const float *__restrict__ val, const int *__restrict__ row_ptr, int m,
                                        float *__restrict__ out) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= m) return;
    float s = 0;
    for (int p = row_ptr[r]; p < row_ptr[r + 1]; ++p) s = fmaf(val[p], val[p], s);
    out[r] = s;
}

// TF32 split x = hi + lo (+ <= 2^-22 |x|): hi = x rounded to TF32, lo = (x - hi) rounded to
// TF32, both with the 13 low mantissa bits cleared so that the tensor core reads exactly
// these values whether it truncates or rounds its FP32 operands.
__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
    unsigned h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    float r = x - hi;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(r));
    lo = __uint_as_float(l);
}

// Row-scaled FP16 split: the row is multiplied by a power of two that puts its largest magnitude in
// [2^14, 2^15), then x*scale = hi + lo (+ <= 2^-24 |x*scale|) with hi, lo FP16 (lo may be subnormal:
// absolute precision 2^-24, i.e. 2^-39 of the row maximum). Products of FP16 values are exact in the
// tensor core's FP32 accumulator, and the epilogue multiplies the sum by the two rows' 1/scale.
__device__ __forceinline__ void row_scale_from_max(float amax, float &scale, float &unscale) {
    const int ex = (int) ((__float_as_uint(amax) >> 23) & 0xffu) - 127;
    int se = (ex == -127) ? 0 : 14 - ex;          // all-zero (or denormal) rows stay unscaled
    se = se < -126 ? -126 : (se > 126 ? 126 : se);
    scale = __uint_as_float((unsigned) (se + 127) << 23);
    unscale = __uint_as_float((unsigned) (127 - se) << 23);
}

__device__ __forceinline__ void split_f16(float xs, __half &hi, __half &lo) {
    hi = __float2half_rn(xs);
    lo = __float2half_rn(xs - __half2float(hi));
}

// plane_kind 1: TF32 words; 2: FP16 halves of the scaled value (off counts elements of the plane).
__device__ __forceinline__ void store_planes(int kind, float *hi, float *lo, size_t off, float v, float scale) {
    if (kind == 2) {
        __half h, l;
        split_f16(v * scale, h, l);
        reinterpret_cast<__half *>(hi)[off] = h;
        reinterpret_cast<__half *>(lo)[off] = l;
    } else {
        float h, l;
        split_tf32(v, h, l);
        hi[off] = h;
        lo[off] = l;
    }
}

// max |v| over the block (every thread calls it once per kernel; blockDim a multiple of 32, <= 1024)
__device__ __forceinline__ float block_max_abs(float v) {
    __shared__ unsigned red[32];
    const unsigned full = 0xffffffffu;
    unsigned b = __reduce_max_sync(full, __float_as_uint(fabsf(v)));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = b;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    b = (int) (threadIdx.x & 31) < nw ? red[threadIdx.x & 31] : 0u;
    return __uint_as_float(__reduce_max_sync(full, b));
}

// Where the staging kernels put a requested row: FP32 W (CUDA-core engine) or the two planes.
struct RowDst {
    float *W, *hi, *lo, *unscale;
    int kind, ld;                  // plane kind (0 = FP32 W) and row length in elements
};

// Planes of all instances: one warp per row; columns d..pld-1 are zero.
__global__ void split_rows_kernel(const float *__restrict__ X, int n, int d, int ld, int kind, int pld,
                                  float *__restrict__ hi, float *__restrict__ lo, float *__restrict__ x_unscale) {
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < n; row += gridDim.x * wpb) {
        const float *x = X + (size_t) row * ld;
        float scale = 1.0f, unscale = 1.0f;
        if (kind == 2) {
            float amax = 0.0f;
            for (int k = lane; k < d; k += 32) amax = fmaxf(amax, fabsf(x[k]));
            amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
            row_scale_from_max(amax, scale, unscale);
            if (lane == 0) x_unscale[row] = unscale;
        }
        for (int k = lane; k < pld; k += 32)
            store_planes(kind, hi, lo, (size_t) row * pld + k, k < d ? x[k] : 0.0f, scale);
    }
}

// ---- gathering the requested rows ----------------------------------------------------------

// Requested row i = X[idx[i]][0..d) (zero padded to the destination's row length); sd_rows[i].
__global__ void gather_rows_dense_kernel(const float *__restrict__ X, int ld, int d, const int *__restrict__ idx,
                                         int m, const float *__restrict__ sd, RowDst dst,
                                         float *__restrict__ sd_rows, const int *__restrict__ m_dev) {
    int i = blockIdx.x;
    if (i >= m || (m_dev && i >= *m_dev)) return;
    const int r = idx[i];
    const int dr = r >= 0 ? d : 0;           // id -1 (an empty working-set slot) is staged as an all-zero row
    const float *x = X + (size_t) (r >= 0 ? r : 0) * ld;
    float scale = 1.0f, unscale = 1.0f;
    if (dst.kind == 2) {
        float amax = 0.0f;
        for (int k = threadIdx.x; k < dr; k += blockDim.x) amax = fmaxf(amax, fabsf(x[k]));
        row_scale_from_max(block_max_abs(amax), scale, unscale);
        if (threadIdx.x == 0) dst.unscale[i] = unscale;
    }
    for (int k = threadIdx.x; k < dst.ld; k += blockDim.x) {
        float v = k < dr ? x[k] : 0.0f;
        if (dst.W) dst.W[(size_t) i * dst.ld + k] = v;
        else store_planes(dst.kind, dst.hi, dst.lo, (size_t) i * dst.ld + k, v, scale);
    }
    if (threadIdx.x == 0) sd_rows[i] = r >= 0 ? sd[r] : 0.0f;
}

// Same for a batch of new dense instances T (m x dt, stride ldt); features >= d are dropped.
__global__ void stage_rows_dense_kernel(const float *__restrict__ T, int ldt, int dt, int d, int m, RowDst dst) {
    int i = blockIdx.x;
    if (i >= m) return;
    const float *x = T + (size_t) i * ldt;
    const int lim = d < dt ? d : dt;
    float scale = 1.0f, unscale = 1.0f;
    if (dst.kind == 2) {
        float amax = 0.0f;
        for (int k = threadIdx.x; k < lim; k += blockDim.x) amax = fmaxf(amax, fabsf(x[k]));
        row_scale_from_max(block_max_abs(amax), scale, unscale);
        if (threadIdx.x == 0) dst.unscale[i] = unscale;
    }
    for (int k = threadIdx.x; k < dst.ld; k += blockDim.x) {
        float v = k < lim ? x[k] : 0.0f;
        if (dst.W) dst.W[(size_t) i * dst.ld + k] = v;
        else store_planes(dst.kind, dst.hi, dst.lo, (size_t) i * dst.ld + k, v, scale);
    }
}

// CSR rows -> zero-initialised dense rows for the dense engines.
__global__ void scatter_csr_to_w_kernel(const float *__restrict__ val, const int *__restrict__ row_ptr,
                                        const int *__restrict__ col, const int *__restrict__ idx, int m, int d,
                                        RowDst dst) {
    int i = blockIdx.x;
    if (i >= m) return;
    int r = idx ? idx[i] : i;
    float scale = 1.0f, unscale = 1.0f;
    if (dst.kind == 2) {
        float amax = 0.0f;
        for (int p = row_ptr[r] + threadIdx.x; p < row_ptr[r + 1]; p += blockDim.x)
            if (col[p] < d) amax = fmaxf(amax, fabsf(val[p]));
        row_scale_from_max(block_max_abs(amax), scale, unscale);
        if (threadIdx.x == 0) dst.unscale[i] = unscale;
    }
    for (int p = row_ptr[r] + threadIdx.x; p < row_ptr[r + 1]; p += blockDim.x) {
        int c = col[p];
        if (c >= d) continue;
        float v = val[p];
        if (dst.W) dst.W[(size_t) i * dst.ld + c] = v;
        else store_planes(dst.kind, dst.hi, dst.lo, (size_t) i * dst.ld + c, v, scale);
    }
}

// CSR engine staging: WT[c * wt_ld + i] = value of feature c in requested row i. WT is kept
// all-zero between calls: `clear` = true writes zeros back at the same places.
__global__ void scatter_csr_to_wt_kernel(const float *__restrict__ val, const int *__restrict__ row_ptr,
                                         const int *__restrict__ col, const int *__restrict__ idx, int m, int d,
                                         int wt_ld, float *__restrict__ WT, const float *__restrict__ sd,
                                         float *__restrict__ sd_rows, bool clear, const int *__restrict__ m_dev) {
    int i = blockIdx.x;
    if (i >= m || (m_dev && i >= *m_dev)) return;
    int r = idx ? idx[i] : i;
    if (r < 0) {                             // an empty working-set slot: an all-zero row
        if (!clear && sd && threadIdx.x == 0) sd_rows[i] = 0.0f;
        return;
    }
    for (int p = row_ptr[r] + threadIdx.x; p < row_ptr[r + 1]; p += blockDim.x) {
        int c = col[p];
        if (c < d) WT[(size_t) c * wt_ld + i] = clear ? 0.0f : val[p];
    }
    if (!clear && sd && threadIdx.x == 0) sd_rows[i] = sd[r];
}

// WT from a dense batch T (m x dt): WT[c * wt_ld + i] = T[i][c] for c < min(d, dt).
__global__ void transpose_dense_to_wt_kernel(const float *__restrict__ T, int ldt, int dt, int d, int m, int wt_ld,
                                             float *__restrict__ WT, bool clear) {
    __shared__ float tile[32][33];
    int c0 = blockIdx.x * 32, i0 = blockIdx.y * 32;
    int tx = threadIdx.x, ty = threadIdx.y;   // 32 x 8
    int lim = d < dt ? d : dt;
    for (int r = ty; r < 32; r += 8) {
        int i = i0 + r, c = c0 + tx;
        tile[r][tx] = (!clear && i < m && c < lim) ? T[(size_t) i * ldt + c] : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        int c = c0 + r, i = i0 + tx;
        if (c < d && i < m) WT[(size_t) c * wt_ld + i] = tile[tx][r];
    }
}

// Operand planes, self dots and 1/scale of the instances ids[0..m) copied out of the kernel matrix's planes
// (row_bytes a multiple of 16).
__global__ void gather_planes_kernel(const float *__restrict__ Xhi, const float *__restrict__ Xlo, size_t row_bytes,
                                     const int *__restrict__ ids, int m, const float *__restrict__ sd,
                                     const float *__restrict__ x_unscale, float *__restrict__ hi,
                                     float *__restrict__ lo, float *__restrict__ sd_out,
                                     float *__restrict__ unscale_out, const int *__restrict__ m_dev) {
    const int i = blockIdx.x;
    if (i >= m || (m_dev && i >= *m_dev)) return;
    const int r = ids[i] >= 0 ? ids[i] : 0;      // an empty slot copies some row; its y = 0 keeps it inert
    const size_t vecs = row_bytes / 16;
    const uint4 *sh = reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(Xhi) + (size_t) r * row_bytes);
    const uint4 *sl = reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(Xlo) + (size_t) r * row_bytes);
    uint4 *dh = reinterpret_cast<uint4 *>(reinterpret_cast<char *>(hi) + (size_t) i * row_bytes);
    uint4 *dl = reinterpret_cast<uint4 *>(reinterpret_cast<char *>(lo) + (size_t) i * row_bytes);
    for (size_t v = threadIdx.x; v < vecs; v += blockDim.x) { dh[v] = sh[v]; dl[v] = sl[v]; }
    if (threadIdx.x == 0) { sd_out[i] = sd[r]; unscale_out[i] = x_unscale ? x_unscale[r] : 1.0f; }
}

// ---- CUDA-core dense engine: out[i][j] = kfn(sum_k W[i][k] X[j][k]) -------------------------
// 64 instances x 64 requested rows per block, 16-wide k slabs, 4x4 outputs per thread.
__global__ void __launch_bounds__(256)
dense_rows_simt_kernel(const float *__restrict__ X, int ldx, int n, const float *__restrict__ W, int ldw, int m_launch,
                       int d_pad, const float *__restrict__ sd, const float *__restrict__ sd_rows, KernelFn fn,
                       float *__restrict__ out, long long ld_out, const int *__restrict__ m_dev,
                       const int *__restrict__ row_slot) {
    __shared__ float xs[16][64 + 4];
    __shared__ float wsm[16][64 + 4];
    const int m = m_dev ? min(m_launch, max(*m_dev, 0)) : m_launch;     // the count found on the device, if any
    const int j0 = blockIdx.x * 64, i0 = blockIdx.y * 64;
    if (i0 >= m) return;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
    const int lr = tid >> 2, lk = (tid & 3) * 4;   // 64 rows x 4 float4 per slab
    for (int k0 = 0; k0 < d_pad; k0 += 16) {
        float4 xv = make_float4(0, 0, 0, 0), wv = make_float4(0, 0, 0, 0);
        if (j0 + lr < n && k0 + lk < d_pad) xv = *reinterpret_cast<const float4 *>(X + (size_t) (j0 + lr) * ldx + k0 + lk);
        if (i0 + lr < m && k0 + lk < d_pad) wv = *reinterpret_cast<const float4 *>(W + (size_t) (i0 + lr) * ldw + k0 + lk);
        __syncthreads();
        xs[lk + 0][lr] = xv.x; xs[lk + 1][lr] = xv.y; xs[lk + 2][lr] = xv.z; xs[lk + 3][lr] = xv.w;
        wsm[lk + 0][lr] = wv.x; wsm[lk + 1][lr] = wv.y; wsm[lk + 2][lr] = wv.z; wsm[lk + 3][lr] = wv.w;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float xa[4], wb[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) { xa[a] = xs[k][tx + 16 * a]; wb[a] = wsm[k][ty + 16 * a]; }
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
                for (int a = 0; a < 4; ++a) acc[b][a] = fmaf(wb[b], xa[a], acc[b][a]);
        }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        int i = i0 + ty + 16 * b;
        if (i >= m) continue;
        float sdi = sd_rows[i];
        const size_t orow = row_slot ? (size_t) row_slot[i] : (size_t) i;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            int j = j0 + tx + 16 * a;
            if (j < n) out[orow * ld_out + j] = apply_kernel(fn, acc[b][a], sdi, sd[j]);
        }
    }
}

// ---- CSR engine ------------------------------------------------------------------------------
// One warp per stored instance; lanes own requested rows c = 4*lane + 128*v (float4 each). For
// every stored entry (col, val) in storage order: acc[c] += val * WT[col][c], the same FP32
// recurrence as the reference's sparse x dense product (kernelmatrix_kernel.cpp:149-160).
// A block covers 32 consecutive instances and transposes its results through shared memory so
// that every requested row receives 128-byte coalesced stores.
template <int NV>
__global__ void __launch_bounds__(256)
csr_rows_kernel(const float *__restrict__ val, const int *__restrict__ row_ptr, const int *__restrict__ col, int n,
                const float *__restrict__ WT, int wt_ld, int m_launch, const float *__restrict__ sd,
                const float *__restrict__ sd_rows, KernelFn fn, float *__restrict__ out, long long ld_out,
                const int *__restrict__ m_dev, const int *__restrict__ row_slot) {
    extern __shared__ float tile[];   // [NV*128][33]
    const int m = m_dev ? min(m_launch, max(*m_dev, 0)) : m_launch;     // the count found on the device, if any
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j0 = blockIdx.x * 32;
    for (int jj = warp; jj < 32; jj += 8) {
        const int j = j0 + jj;
        float4 acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] = make_float4(0, 0, 0, 0);
        if (j < n) {
            const int b = row_ptr[j], e = row_ptr[j + 1];
            for (int p0 = b; p0 < e; p0 += 32) {
                int cc = 0;
                float vv = 0;
                if (p0 + lane < e) { cc = col[p0 + lane]; vv = val[p0 + lane]; }
                const int cnt = min(32, e - p0);
                for (int t = 0; t < cnt; ++t) {
                    const int c = __shfl_sync(0xffffffffu, cc, t);
                    const float x = __shfl_sync(0xffffffffu, vv, t);
                    const float4 *w = reinterpret_cast<const float4 *>(WT + (size_t) c * wt_ld) + lane;
#pragma unroll
                    for (int v = 0; v < NV; ++v) {
                        float4 wv = __ldg(w + 32 * v);
                        acc[v].x = fmaf(x, wv.x, acc[v].x);
                        acc[v].y = fmaf(x, wv.y, acc[v].y);
                        acc[v].z = fmaf(x, wv.z, acc[v].z);
                        acc[v].w = fmaf(x, wv.w, acc[v].w);
                    }
                }
            }
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int c = 128 * v + 4 * lane;
            tile[(c + 0) * 33 + jj] = acc[v].x;
            tile[(c + 1) * 33 + jj] = acc[v].y;
            tile[(c + 2) * 33 + jj] = acc[v].z;
            tile[(c + 3) * 33 + jj] = acc[v].w;
        }
    }
    __syncthreads();
    const int j = j0 + lane;
    const float sdj = j < n ? sd[j] : 0.0f;
    if ((ld_out & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && j0 + 32 <= n) {
        // four consecutive instances of one row per thread, one 16-byte store: a warp covers four rows
        const int jq = 4 * (lane & 7);
        const float s0 = __shfl_sync(0xffffffffu, sdj, jq), s1 = __shfl_sync(0xffffffffu, sdj, jq + 1),
                    s2 = __shfl_sync(0xffffffffu, sdj, jq + 2), s3 = __shfl_sync(0xffffffffu, sdj, jq + 3);
#pragma unroll 2
        for (int c = 4 * warp + (lane >> 3); c < m; c += 32) {
            const float *tr = tile + c * 33 + jq;
            const float sr = sd_rows[c];
            const size_t orow = row_slot ? (size_t) row_slot[c] : (size_t) c;
            float4 o;
            o.x = apply_kernel(fn, tr[0], sr, s0); o.y = apply_kernel(fn, tr[1], sr, s1);
            o.z = apply_kernel(fn, tr[2], sr, s2); o.w = apply_kernel(fn, tr[3], sr, s3);
            *reinterpret_cast<float4 *>(out + orow * ld_out + j0 + jq) = o;
        }
        return;
    }
    for (int c = warp; c < m; c += 8) {
        const size_t orow = row_slot ? (size_t) row_slot[c] : (size_t) c;
        if (j < n) out[orow * ld_out + j] = apply_kernel(fn, tile[c * 33 + lane], sd_rows[c], sdj);
    }
}

// ---- CSR engine for few features: the panel in shared memory ---------------------------------------
// csr_rows_kernel reads a 2 KB panel row from L2 for every stored entry; with d features the panel is only
// d x 1 KB per 256 requested rows, which fits in shared memory for d <= CSR_SMEM_MAX_D. A block then loads
// its 256-row part of the panel once and sweeps instance tiles with it (grid: blocks x parts, every block a
// strided share of the 32-instance tiles): a stored entry costs two 16-byte shared-memory loads and eight
// multiply-adds per lane instead of a trip to L2. Same FP32 recurrence in storage order per (row, instance),
// so the values are those of csr_rows_kernel bit for bit. Results go through a double-buffered transposed
// tile so that every requested row receives 128-byte coalesced stores.
constexpr int CSR_SMEM_THREADS = 512, CSR_SMEM_PART = 256, CSR_SMEM_TILE = CSR_SMEM_PART * 33;
constexpr int CSR_SMEM_MAX_D = (227 * 1024 - 2 * CSR_SMEM_TILE * 4 - 2 * CSR_SMEM_PART * 4 - 64) / (CSR_SMEM_PART * 4);

__global__ void __launch_bounds__(CSR_SMEM_THREADS, 1)
csr_rows_smem_kernel(const float *__restrict__ val, const int *__restrict__ row_ptr, const int *__restrict__ col, int n,
                     int d, const float *__restrict__ WT, int wt_ld, int m_launch, const float *__restrict__ sd,
                     const float *__restrict__ sd_rows, KernelFn fn, float *__restrict__ out, long long ld_out,
                     const int *__restrict__ m_dev, const int *__restrict__ row_slot) {
    extern __shared__ __align__(16) float csr_sm[];          // panel [d][256] | tile [2][256][33]
    const int m = m_dev ? min(m_launch, max(*m_dev, 0)) : m_launch;     // the count found on the device, if any
    const int c0 = blockIdx.y * CSR_SMEM_PART;
    if (c0 >= m) return;
    const int mh = min(CSR_SMEM_PART, m - c0);
    float4 *panel4 = reinterpret_cast<float4 *>(csr_sm);
    float *tiles = csr_sm + (size_t) d * CSR_SMEM_PART;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __shared__ int orow_sm[CSR_SMEM_PART];
    __shared__ float sdr_sm[CSR_SMEM_PART];
    if (tid < mh) {
        orow_sm[tid] = row_slot ? row_slot[c0 + tid] : c0 + tid;
        sdr_sm[tid] = sd_rows[c0 + tid];
    }
    for (int i = tid; i < d * (CSR_SMEM_PART / 4); i += CSR_SMEM_THREADS) {
        const int c = i / (CSR_SMEM_PART / 4), v = i % (CSR_SMEM_PART / 4);
        panel4[i] = __ldg(reinterpret_cast<const float4 *>(WT + (size_t) c * wt_ld + c0) + v);
    }
    __syncthreads();
    const int n_tiles = (n + 31) / 32;
    const bool vec_ok = (ld_out & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    constexpr int PER_WARP = 32 / (CSR_SMEM_THREADS / 32);        // instances of a tile per warp
    // The CSR entries of the next tile's instances are fetched (row bounds, then the first 32 entries) while
    // this tile is computed: the two dependent trips to memory per instance stay off the critical path.
    int nb[PER_WARP], ne[PER_WARP], ncc[PER_WARP];
    float nvv[PER_WARP], nsd = 0.0f;
    auto fetch = [&](int ti) {
#pragma unroll
        for (int u = 0; u < PER_WARP; ++u) {
            const int j = ti * 32 + warp + u * (CSR_SMEM_THREADS / 32);
            nb[u] = ne[u] = 0; ncc[u] = 0; nvv[u] = 0.0f;
            if (ti < n_tiles && j < n) { nb[u] = row_ptr[j]; ne[u] = row_ptr[j + 1]; }
        }
#pragma unroll
        for (int u = 0; u < PER_WARP; ++u)
            if (nb[u] + lane < ne[u]) { ncc[u] = col[nb[u] + lane]; nvv[u] = val[nb[u] + lane]; }
        const int j = ti * 32 + lane;
        nsd = (ti < n_tiles && j < n) ? sd[j] : 0.0f;
    };
    fetch(blockIdx.x);
    int buf = 0;
    for (int ti = blockIdx.x; ti < n_tiles; ti += gridDim.x, buf ^= 1) {
        const int j0 = ti * 32;
        float *T = tiles + buf * CSR_SMEM_TILE;
        int cb[PER_WARP], ce[PER_WARP], ccc[PER_WARP];
        float cvv[PER_WARP];
#pragma unroll
        for (int u = 0; u < PER_WARP; ++u) { cb[u] = nb[u]; ce[u] = ne[u]; ccc[u] = ncc[u]; cvv[u] = nvv[u]; }
        const float sdj = nsd;
        fetch(ti + gridDim.x);
#pragma unroll
        for (int u = 0; u < PER_WARP; ++u) {
            const int jj = warp + u * (CSR_SMEM_THREADS / 32);
            // rows c0 + 4 * lane + 0..3 and c0 + 128 + 4 * lane + 0..3: a warp's 16-byte loads cover 512 contiguous bytes
            float4 a0 = make_float4(0, 0, 0, 0), a1 = make_float4(0, 0, 0, 0);
            for (int p0 = cb[u]; p0 < ce[u]; p0 += 32) {
                int cc = ccc[u];
                float vv = cvv[u];
                if (p0 != cb[u]) {                  // beyond the prefetched entries
                    cc = 0; vv = 0;
                    if (p0 + lane < ce[u]) { cc = col[p0 + lane]; vv = val[p0 + lane]; }
                }
                const int cnt = min(32, ce[u] - p0);
                int t = 0;
                // four stored entries at a time: their panel loads are independent, the sums keep the storage order
                for (; t + 4 <= cnt; t += 4) {
                    float x[4];
                    float4 w0[4], w1[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int c = __shfl_sync(0xffffffffu, cc, t + k);
                        x[k] = __shfl_sync(0xffffffffu, vv, t + k);
                        const float4 *w = panel4 + (size_t) c * (CSR_SMEM_PART / 4) + lane;
                        w0[k] = w[0]; w1[k] = w[32];
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        a0.x = fmaf(x[k], w0[k].x, a0.x); a0.y = fmaf(x[k], w0[k].y, a0.y);
                        a0.z = fmaf(x[k], w0[k].z, a0.z); a0.w = fmaf(x[k], w0[k].w, a0.w);
                        a1.x = fmaf(x[k], w1[k].x, a1.x); a1.y = fmaf(x[k], w1[k].y, a1.y);
                        a1.z = fmaf(x[k], w1[k].z, a1.z); a1.w = fmaf(x[k], w1[k].w, a1.w);
                    }
                }
                for (; t < cnt; ++t) {
                    const int c = __shfl_sync(0xffffffffu, cc, t);
                    const float x = __shfl_sync(0xffffffffu, vv, t);
                    const float4 *w = panel4 + (size_t) c * (CSR_SMEM_PART / 4) + lane;
                    const float4 w0 = w[0], w1 = w[32];
                    a0.x = fmaf(x, w0.x, a0.x); a0.y = fmaf(x, w0.y, a0.y);
                    a0.z = fmaf(x, w0.z, a0.z); a0.w = fmaf(x, w0.w, a0.w);
                    a1.x = fmaf(x, w1.x, a1.x); a1.y = fmaf(x, w1.y, a1.y);
                    a1.z = fmaf(x, w1.z, a1.z); a1.w = fmaf(x, w1.w, a1.w);
                }
            }
            // row 4 * lane + k (+ 128) sits in tile row 32 * k + lane (+ 128): a warp's stores hit 32 banks each
            T[(0 * 32 + lane) * 33 + jj] = a0.x; T[(1 * 32 + lane) * 33 + jj] = a0.y;
            T[(2 * 32 + lane) * 33 + jj] = a0.z; T[(3 * 32 + lane) * 33 + jj] = a0.w;
            T[(4 * 32 + lane) * 33 + jj] = a1.x; T[(5 * 32 + lane) * 33 + jj] = a1.y;
            T[(6 * 32 + lane) * 33 + jj] = a1.z; T[(7 * 32 + lane) * 33 + jj] = a1.w;
        }
        __syncthreads();
        // (the other buffer is written next; this one again only after the next barrier, which every warp
        // reaches after it has read its rows here)
        if (vec_ok && j0 + 32 <= n) {
            // four consecutive instances of one row per thread, one 16-byte store: a warp covers four rows
            const int jq = 4 * (lane & 7);
            const float s0 = __shfl_sync(0xffffffffu, sdj, jq), s1 = __shfl_sync(0xffffffffu, sdj, jq + 1),
                        s2 = __shfl_sync(0xffffffffu, sdj, jq + 2), s3 = __shfl_sync(0xffffffffu, sdj, jq + 3);
#pragma unroll 2
            for (int c = 4 * warp + (lane >> 3); c < mh; c += 4 * (CSR_SMEM_THREADS / 32)) {
                const float *tr = T + ((((c >> 7) << 2) + (c & 3)) * 32 + ((c & 127) >> 2)) * 33 + jq;
                const float sr = sdr_sm[c];
                float4 o;
                o.x = apply_kernel(fn, tr[0], sr, s0); o.y = apply_kernel(fn, tr[1], sr, s1);
                o.z = apply_kernel(fn, tr[2], sr, s2); o.w = apply_kernel(fn, tr[3], sr, s3);
                *reinterpret_cast<float4 *>(out + (size_t) orow_sm[c] * ld_out + j0 + jq) = o;
            }
        } else {
            const int j = j0 + lane;
            for (int c = warp; c < mh; c += CSR_SMEM_THREADS / 32) {
                const float dot = T[((((c >> 7) << 2) + (c & 3)) * 32 + ((c & 127) >> 2)) * 33 + lane];
                if (j < n) out[(size_t) orow_sm[c] * ld_out + j] = apply_kernel(fn, dot, sdr_sm[c], sdj);
            }
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------

static tsvm_status ensure_scratch(tsvm_km *km, int m) {
    if (m <= km->w_cap) return TSVM_OK;
    int cap = 128;
    while (cap < m) cap *= 2;
    pool_free_many({km->W, km->Whi, km->Wlo, km->WT, km->sd_rows, km->w_unscale});
    km->W = km->Whi = km->Wlo = km->WT = km->sd_rows = km->w_unscale = nullptr;
    km->w_cap = 0;
    TSVM_TRY(dev_alloc(&km->sd_rows, (size_t) cap));
    if (km->dense) {
        // either plane kind fits cap x d_pad words: round_up(d, 8) halves <= d_pad floats
        TSVM_TRY(dev_alloc(&km->w_unscale, (size_t) cap));
        TSVM_TRY(dev_alloc(&km->W, (size_t) cap * km->d_pad));
        TSVM_TRY(dev_alloc(&km->Whi, (size_t) cap * km->d_pad));
        TSVM_TRY(dev_alloc(&km->Wlo, (size_t) cap * km->d_pad));
    } else {
        km->wt_ld = cap;
        TSVM_TRY(dev_alloc(&km->WT, (size_t) km->d * cap));
        TSVM_CUDA(cudaMemset(km->WT, 0, sizeof(float) * (size_t) km->d * cap));
    }
    km->w_cap = cap;
    return TSVM_OK;
}

// engine: 0 = automatic, 1 = CUDA cores, 3 (and its old alias 2) = tensor cores on TF32 planes, 4 = tensor
// cores on row-scaled FP16 planes (what "automatic" picks for d_pad > 32); both tensor forms run on CTA pairs
static inline bool use_tensor_engine(const tsvm_km *km) {
    return km->engine >= 2 || (km->engine == 0 && km->d_pad > 32);
}
static inline int wanted_plane_kind(const tsvm_km *km) {
    if (!km->dense || !use_tensor_engine(km)) return 0;
    return (km->engine == 2 || km->engine == 3) ? 1 : 2;
}

// Builds the planes the selected engine reads, once; a change of engine rebuilds them.
static tsvm_status ensure_planes(tsvm_km *km, cudaStream_t st) {
    const int kind = wanted_plane_kind(km);
    if (kind == 0 || kind == km->plane_kind) return TSVM_OK;
    pool_free_many({km->Xhi, km->Xlo});
    km->Xhi = km->Xlo = nullptr;
    km->plane_kind = 0;
    km->plane_ld = kind == 1 ? km->d_pad : (km->d + 7) & ~7;
    const size_t words = kind == 1 ? (size_t) km->n * km->plane_ld : ((size_t) km->n * km->plane_ld + 1) / 2;
    TSVM_TRY(dev_alloc(&km->Xhi, words));
    TSVM_TRY(dev_alloc(&km->Xlo, words));
    if (!km->x_unscale) TSVM_TRY(dev_alloc(&km->x_unscale, (size_t) km->n));
    TSVM_LAUNCH(split_rows_kernel, 148 * 8, 256, 0, st, km->X, km->n, km->d, km->ldx, kind, km->plane_ld, km->Xhi,
                km->Xlo, km->x_unscale);
    km->plane_kind = kind;
    return TSVM_OK;
}

static inline RowDst row_dst(const tsvm_km *km) {
    if (use_tensor_engine(km)) return RowDst{nullptr, km->Whi, km->Wlo, km->w_unscale, km->plane_kind, km->plane_ld};
    return RowDst{km->W, nullptr, nullptr, nullptr, 0, km->d_pad};
}
static inline size_t row_dst_bytes(const RowDst &r, int m) {
    return (size_t) m * r.ld * (r.kind == 2 ? sizeof(__half) : sizeof(float));
}

static tsvm_status finish_create(tsvm_km *km, cudaStream_t st) {
    TSVM_TRY(dev_alloc(&km->self_dot, (size_t) km->n));
    TSVM_TRY(dev_alloc(&km->diag, (size_t) km->n));
    TSVM_TRY(dev_alloc(&km->status_dev, 4));
    TSVM_CUDA(cudaMemsetAsync(km->status_dev, 0, 4 * sizeof(int), st));
    TSVM_TRY(pinned_alloc((void **) &km->status_host, 4 * sizeof(int)));
    const int blocks = ceil_div((long long) km->n * 32, 256);
    if (km->dense)
        TSVM_LAUNCH(self_dot_dense_kernel, blocks, 256, 0, st, km->X, km->n, km->d, km->ldx, km->self_dot);
    else
        TSVM_LAUNCH(self_dot_csr_kernel, blocks, 256, 0, st, km->val, km->row_ptr, km->n, km->self_dot);
    TSVM_LAUNCH(diag_kernel, ceil_div(km->n, 256), 256, 0, st, km->self_dot, km->n, km->fn, km->diag);
    return ensure_planes(km, st);
}

// TSVM_CSR_SMEM=0 keeps the L2-panel engine for every CSR matrix (used to compare the two engines)
static bool csr_smem_engine_allowed() {
    static const bool on = [] { const char *e = getenv("TSVM_CSR_SMEM"); return !e || atoi(e) != 0; }();
    return on;
}

// A set of stored instances the CSR engines sweep: the kernel matrix's own, or a gathered subset of them.
struct CsrView {
    const float *val;
    const int *row_ptr, *col;
    int n;
    const float *sd;                // self dots of the instances
};

// Kernel rows of the m requested rows staged in `panel` (feature-major, row stride km->wt_ld; self dots in
// sd_rows) against the instances of X. spare_sms: SMs the persistent engine leaves free.
static tsvm_status csr_engine_launch(tsvm_km *km, const CsrView &X, const float *panel, const float *sd_rows, int m,
                                     float *out, long long ld_out, const int *m_dev, const int *row_slot, int spare_sms,
                                     cudaStream_t st) {
    if (km->d <= CSR_SMEM_MAX_D && csr_smem_engine_allowed()) {
        // few features: the panel of 256 requested rows fits in shared memory
        const size_t smem = ((size_t) km->d * CSR_SMEM_PART + 2 * CSR_SMEM_TILE) * sizeof(float);
        TSVM_ONCE_PER_DEVICE(TSVM_CUDA(cudaFuncSetAttribute(csr_rows_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                            (int) (((size_t) CSR_SMEM_MAX_D * CSR_SMEM_PART + 2 * CSR_SMEM_TILE) * sizeof(float)))));
        const int parts = ceil_div(m, CSR_SMEM_PART);
        int sms = 148;
        {
            int dev = 0;
            TSVM_CUDA(cudaGetDevice(&dev));
            TSVM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        }
        sms = sms - spare_sms > 0 ? sms - spare_sms : 1;
        int bx = sms / parts > 0 ? sms / parts : 1;
        const int n_tiles = ceil_div(X.n, 32);
        if (bx > n_tiles) bx = n_tiles;
        TSVM_LAUNCH(csr_rows_smem_kernel, dim3(bx, parts), CSR_SMEM_THREADS, smem, st, X.val, X.row_ptr, X.col, X.n, km->d,
                    panel, km->wt_ld, m, X.sd, sd_rows, km->fn, out, ld_out, m_dev, row_slot);
        return TSVM_OK;
    }
    const int nv = ceil_div(m, 128);
    const int grid = ceil_div(X.n, 32);
#define CSR_CASE(NV)                                                                                             \
    {                                                                                                            \
        size_t smem = (size_t) (NV) * 128 * 33 * sizeof(float);                                                  \
        TSVM_CUDA(cudaFuncSetAttribute(csr_rows_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                       (int) smem));                                                             \
        TSVM_LAUNCH(csr_rows_kernel<NV>, grid, 256, smem, st, X.val, X.row_ptr, X.col, X.n, panel, km->wt_ld, m, \
                    X.sd, sd_rows, km->fn, out, ld_out, m_dev, row_slot);                                        \
    }
    if (nv <= 1) CSR_CASE(1)
    else if (nv <= 2) CSR_CASE(2)
    else if (nv <= 4) CSR_CASE(4)
    else if (nv <= 8) CSR_CASE(8)
    else { set_error("CSR engine handles at most 1024 rows per call, got %d", m); return TSVM_ERR_INVALID; }
#undef CSR_CASE
    return TSVM_OK;
}

static tsvm_status rows_common(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st) {
    // W / WT and sd_rows are staged; run the engine.
    if (km->dense) {
        if (use_tensor_engine(km)) return launch_dense_tc(km, m, out, ld_out, st);
        dim3 grid(ceil_div(km->n, 64), ceil_div(m, 64));
        TSVM_LAUNCH(dense_rows_simt_kernel, grid, 256, 0, st, km->X, km->ldx, km->n, km->W, km->d_pad, m, km->d_pad,
                    km->self_dot, km->sd_rows, km->fn, out, ld_out, km->rows_m_dev, km->rows_slot_dev);
        return TSVM_OK;
    }
    return csr_engine_launch(km, CsrView{km->val, km->row_ptr, km->col, km->n, km->self_dot}, km->WT, km->sd_rows, m, out,
                             ld_out, km->rows_m_dev, km->rows_slot_dev, 0, st);
}

// ---- pieces of tsvm_km_rows_by_index for callers that overlap them (the solver) -------------------
tsvm_status launch_dense_tc2_on(tsvm_km *km, const InstancePlanes &X, int m, float *out, long long ld_out,
                                cudaStream_t st);   // dense_tc2.cu

// True when kernel rows of this matrix run on the CTA-pair tensor engine, whose requested-row staging and
// launch can be issued separately and against a caller-chosen subset of instances.
bool km_pair_engine(tsvm_km *km, cudaStream_t st) {
    if (!km->dense || !use_tensor_engine(km)) return false;
    return ensure_planes(km, st) == TSVM_OK && km->plane_kind != 0;
}

size_t km_plane_row_bytes(const tsvm_km *km) {
    return (size_t) km->plane_ld * (km->plane_kind == 2 ? sizeof(__half) : sizeof(float));
}

tsvm_status km_stage_rows_by_index(tsvm_km *km, const int *idx_dev, int q, cudaStream_t st) {
    TSVM_TRY(ensure_scratch(km, q));
    TSVM_TRY(ensure_planes(km, st));
    TSVM_LAUNCH(gather_rows_dense_kernel, q, 256, 0, st, km->X, km->ldx, km->d, idx_dev, q, km->self_dot, row_dst(km),
                km->sd_rows, km->rows_m_dev);
    return TSVM_OK;
}

tsvm_status km_rows_staged(tsvm_km *km, int q, float *out, long long ld_out, cudaStream_t st) {
    return rows_common(km, q, out, ld_out, st);
}

tsvm_status km_gather_planes(tsvm_km *km, const int *ids_dev, int m, const int *m_dev, float *hi, float *lo, float *sd,
                             float *unscale, cudaStream_t st) {
    TSVM_LAUNCH(gather_planes_kernel, m, 128, 0, st, km->Xhi, km->Xlo, km_plane_row_bytes(km), ids_dev, m,
                km->self_dot, km->plane_kind == 2 ? km->x_unscale : nullptr, hi, lo, sd, unscale, m_dev);
    return TSVM_OK;
}

tsvm_status km_rows_staged_on(tsvm_km *km, const InstancePlanes &X, int q, float *out, long long ld_out,
                              cudaStream_t st) {
    return launch_dense_tc2_on(km, X, q, out, ld_out, st);
}

tsvm_status launch_dense_tc2_planes(tsvm_km *km, const InstancePlanes &X, const RowPlanes &W, int m, float *out,
                                    long long ld_out, cudaStream_t st);   // dense_tc2.cu

tsvm_status km_rows_planes_on(tsvm_km *km, const InstancePlanes &X, const RowPlanes &W, int q, float *out,
                              long long ld_out, cudaStream_t st) {
    return launch_dense_tc2_planes(km, X, W, q, out, ld_out, st);
}

// Stages m explicit feature rows (m x n_features, stride ldt) with their self dots as the requested rows.
tsvm_status km_stage_rows_features(tsvm_km *km, const float *T_dev, int ldt, const float *sd_T_dev, int m,
                                   cudaStream_t st) {
    TSVM_TRY(ensure_scratch(km, m));
    TSVM_TRY(ensure_planes(km, st));
    TSVM_CUDA(cudaMemcpyAsync(km->sd_rows, sd_T_dev, sizeof(float) * m, cudaMemcpyDeviceToDevice, st));
    TSVM_LAUNCH(stage_rows_dense_kernel, m, 256, 0, st, T_dev, ldt, km->d, km->d, m, row_dst(km));
    return TSVM_OK;
}

// Stages mm new instances as the requested rows of a dense kernel matrix (self dots accumulated in storage
// order as kernelmatrix.cpp:288-296 does, rows in the engine's operand form): the first half of
// tsvm_km_rows_by_instances_*, shared with the fused prediction.
tsvm_status km_stage_instances_dense(tsvm_km *km, const float *T, int mm, int dt, int ldt, cudaStream_t st) {
    TSVM_TRY(ensure_scratch(km, mm));
    TSVM_LAUNCH(self_dot_seq_dense_kernel, ceil_div(mm, 128), 128, 0, st, T, mm, dt, ldt, km->sd_rows);
    TSVM_TRY(ensure_planes(km, st));
    TSVM_LAUNCH(stage_rows_dense_kernel, mm, 256, 0, st, T, ldt, dt, km->d, mm, row_dst(km));
    return TSVM_OK;
}

tsvm_status km_stage_instances_csr(tsvm_km *km, const float *tval, const int *rp, const int *tcol, int mm,
                                   cudaStream_t st) {
    TSVM_TRY(ensure_scratch(km, mm));
    TSVM_LAUNCH(self_dot_seq_csr_kernel, ceil_div(mm, 128), 128, 0, st, tval, rp, mm, km->sd_rows);
    TSVM_TRY(ensure_planes(km, st));
    const RowDst dst = row_dst(km);
    if (dst.W) TSVM_CUDA(cudaMemsetAsync(dst.W, 0, row_dst_bytes(dst, mm), st));
    else {
        TSVM_CUDA(cudaMemsetAsync(dst.hi, 0, row_dst_bytes(dst, mm), st));
        TSVM_CUDA(cudaMemsetAsync(dst.lo, 0, row_dst_bytes(dst, mm), st));
    }
    TSVM_LAUNCH(scatter_csr_to_w_kernel, mm, 128, 0, st, tval, rp, tcol, (const int *) nullptr, mm, km->d, dst);
    return TSVM_OK;
}

}  // namespace tsvm

using namespace tsvm;

extern "C" {

const char *tsvm_last_error(void) { return tsvm::g_err; }
int tsvm_abi_version(void) { return 2; }
void tsvm_release_cached_memory(void) { tsvm::pool_release(); }

tsvm_status tsvm_km_create_dense(const float *X, int n, int d, int ld, int loc, int kernel_type, int degree,
                                 float gamma, float coef0, void *stream, tsvm_km **out) {
    TSVM_REQUIRE(out && X && n > 0 && d > 0 && ld >= d, "km_create_dense: bad arguments (n=%d d=%d ld=%d)", n, d, ld);
    TSVM_REQUIRE(kernel_type >= TSVM_LINEAR && kernel_type <= TSVM_PRECOMPUTED, "unknown kernel type %d", kernel_type);
    cudaStream_t st = (cudaStream_t) stream;
    tsvm_km *km = new tsvm_km;
    *out = nullptr;
    km->n = n; km->d = d; km->nnz = (long long) n * d; km->dense = true;
    km->fn = KernelFn{kernel_type, degree, gamma, coef0};
    km->d_pad = (d + 3) & ~3;
    tsvm_status s = TSVM_OK;
    bool in_place = loc == TSVM_DEVICE && (d % 4 == 0) && (ld % 4 == 0) && (((uintptr_t) X & 15) == 0) && ld >= km->d_pad;
    if (in_place) { km->X = X; km->ldx = ld; }
    else {
        km->ldx = km->d_pad;
        s = dev_alloc(&km->X_owned, (size_t) n * km->d_pad);
        if (s == TSVM_OK && km->d_pad != d) {
            cudaError_t e = cudaMemsetAsync(km->X_owned, 0, sizeof(float) * (size_t) n * km->d_pad, st);
            if (e != cudaSuccess) { set_error("memset failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
        }
        if (s == TSVM_OK) {
            cudaError_t e = cudaMemcpy2DAsync(km->X_owned, sizeof(float) * km->d_pad, X, sizeof(float) * ld,
                                              sizeof(float) * d, n,
                                              loc == TSVM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                              st);
            if (e != cudaSuccess) { set_error("copy of X failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
        }
        km->X = km->X_owned;
    }
    if (s == TSVM_OK) s = finish_create(km, st);
    if (s != TSVM_OK) { tsvm_km_destroy(km); return s; }
    *out = km;
    return TSVM_OK;
}

tsvm_status tsvm_km_create_csr(const float *val, const int *row_ptr, const int *col, int n, int d, int loc,
                               int kernel_type, int degree, float gamma, float coef0, void *stream, tsvm_km **out) {
    TSVM_REQUIRE(out && row_ptr && n > 0 && d > 0, "km_create_csr: bad arguments (n=%d d=%d)", n, d);
    TSVM_REQUIRE(kernel_type >= TSVM_LINEAR && kernel_type <= TSVM_PRECOMPUTED, "unknown kernel type %d", kernel_type);
    cudaStream_t st = (cudaStream_t) stream;
    tsvm_km *km = new tsvm_km;
    *out = nullptr;
    km->n = n; km->d = d; km->dense = false;
    km->fn = KernelFn{kernel_type, degree, gamma, coef0};
    tsvm_status s = TSVM_OK;
    int last = 0;
    if (loc == TSVM_HOST) last = row_ptr[n];
    else if (cudaMemcpy(&last, row_ptr + n, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) s = TSVM_ERR_CUDA;
    km->nnz = last;
    if (s == TSVM_OK && loc == TSVM_DEVICE) { km->val = val; km->row_ptr = row_ptr; km->col = col; }
    else if (s == TSVM_OK) {
        s = dev_alloc(&km->val_owned, (size_t) last);
        if (s == TSVM_OK) s = dev_alloc(&km->col_owned, (size_t) last);
        if (s == TSVM_OK) s = dev_alloc(&km->row_ptr_owned, (size_t) n + 1);
        if (s == TSVM_OK) {
            cudaError_t e = cudaMemcpyAsync(km->val_owned, val, sizeof(float) * last, cudaMemcpyHostToDevice, st);
            if (e == cudaSuccess) e = cudaMemcpyAsync(km->col_owned, col, sizeof(int) * last, cudaMemcpyHostToDevice, st);
            if (e == cudaSuccess)
                e = cudaMemcpyAsync(km->row_ptr_owned, row_ptr, sizeof(int) * ((size_t) n + 1), cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) { set_error("copy of CSR failed: %s", cudaGetErrorString(e)); s = TSVM_ERR_CUDA; }
        }
        km->val = km->val_owned; km->col = km->col_owned; km->row_ptr = km->row_ptr_owned;
    }
    if (s == TSVM_OK) s = finish_create(km, st);
    if (s != TSVM_OK) { tsvm_km_destroy(km); return s; }
    *out = km;
    return TSVM_OK;
}

void tsvm_km_destroy(tsvm_km *km) {
    if (!km) return;
    pool_free_many({km->X_owned, km->Xhi, km->Xlo, km->x_unscale, km->w_unscale, km->val_owned, km->row_ptr_owned,
                    km->col_owned, km->self_dot, km->diag, km->W, km->Whi, km->Wlo, km->WT, km->sd_rows,
                    km->status_dev});
    if (km->status_host) pinned_free(km->status_host);
    delete km;
}

int tsvm_km_n_instances(const tsvm_km *km) { return km ? km->n : 0; }
int tsvm_km_n_features(const tsvm_km *km) { return km ? km->d : 0; }
long long tsvm_km_nnz(const tsvm_km *km) { return km ? km->nnz : 0; }
int tsvm_km_is_dense(const tsvm_km *km) { return km && km->dense; }
const float *tsvm_km_diag_dev(const tsvm_km *km) { return km ? km->diag : nullptr; }
const float *tsvm_km_self_dot_dev(const tsvm_km *km) { return km ? km->self_dot : nullptr; }

tsvm_status tsvm_km_set_dense_engine(tsvm_km *km, int engine) {
    TSVM_REQUIRE(km && engine >= 0 && engine <= 4, "set_dense_engine: bad arguments");
    km->engine = engine;
    return TSVM_OK;
}

tsvm_status tsvm_km_rows_by_index(tsvm_km *km, const int *idx_dev, int q, float *out_dev, long long ld_out,
                                  void *stream) {
    TSVM_REQUIRE(km && idx_dev && out_dev && q > 0 && ld_out >= km->n, "rows_by_index: bad arguments (q=%d)", q);
    cudaStream_t st = (cudaStream_t) stream;
    TSVM_TRY(ensure_scratch(km, q));
    if (km->dense) {
        TSVM_TRY(ensure_planes(km, st));
        TSVM_LAUNCH(gather_rows_dense_kernel, q, 256, 0, st, km->X, km->ldx, km->d, idx_dev, q, km->self_dot,
                    row_dst(km), km->sd_rows, km->rows_m_dev);
        return rows_common(km, q, out_dev, ld_out, st);
    }
    TSVM_REQUIRE(q <= 1024, "CSR engine handles at most 1024 rows per call, got %d", q);
    TSVM_LAUNCH(scatter_csr_to_wt_kernel, q, 128, 0, st, km->val, km->row_ptr, km->col, idx_dev, q, km->d, km->wt_ld,
                km->WT, km->self_dot, km->sd_rows, false, km->rows_m_dev);
    TSVM_TRY(rows_common(km, q, out_dev, ld_out, st));
    TSVM_LAUNCH(scatter_csr_to_wt_kernel, q, 128, 0, st, km->val, km->row_ptr, km->col, idx_dev, q, km->d, km->wt_ld,
                km->WT, nullptr, nullptr, true, km->rows_m_dev);
    return TSVM_OK;
}

tsvm_status tsvm_km_rows_by_instances_dense(tsvm_km *km, const float *T_dev, int m, int dt, int ldt, float *out_dev,
                                            long long ld_out, void *stream) {
    TSVM_REQUIRE(km && T_dev && out_dev && m > 0 && dt > 0 && ldt >= dt && ld_out >= km->n,
                 "rows_by_instances_dense: bad arguments");
    cudaStream_t st = (cudaStream_t) stream;
    const int chunk = km->dense ? 4096 : 1024;
    for (int r0 = 0; r0 < m; r0 += chunk) {
        const int mm = min(chunk, m - r0);
        const float *T = T_dev + (size_t) r0 * ldt;
        float *o = out_dev + (size_t) r0 * ld_out;
        if (km->dense) {
            TSVM_TRY(km_stage_instances_dense(km, T, mm, dt, ldt, st));
            TSVM_TRY(rows_common(km, mm, o, ld_out, st));
        } else {
            TSVM_TRY(ensure_scratch(km, mm));
            TSVM_LAUNCH(self_dot_seq_dense_kernel, ceil_div(mm, 128), 128, 0, st, T, mm, dt, ldt, km->sd_rows);
            dim3 grid(ceil_div(km->d, 32), ceil_div(mm, 32)), block(32, 8);
            TSVM_LAUNCH(transpose_dense_to_wt_kernel, grid, block, 0, st, T, ldt, dt, km->d, mm, km->wt_ld, km->WT,
                        false);
            TSVM_TRY(rows_common(km, mm, o, ld_out, st));
            TSVM_LAUNCH(transpose_dense_to_wt_kernel, grid, block, 0, st, T, ldt, dt, km->d, mm, km->wt_ld, km->WT,
                        true);
        }
    }
    return TSVM_OK;
}

tsvm_status tsvm_km_rows_for_features_dense(tsvm_km *km, const float *T_dev, int ldt, const float *sd_T_dev, int m,
                                            float *out_dev, long long ld_out, void *stream) {
    TSVM_REQUIRE(km && km->dense && T_dev && sd_T_dev && out_dev && m > 0 && ldt >= km->d && ld_out >= km->n,
                 "rows_for_features_dense: bad arguments (dense kernel matrix required)");
    cudaStream_t st = (cudaStream_t) stream;
    for (int r0 = 0; r0 < m; r0 += 4096) {
        const int mm = min(4096, m - r0);
        TSVM_TRY(ensure_scratch(km, mm));
        TSVM_CUDA(cudaMemcpyAsync(km->sd_rows, sd_T_dev + r0, sizeof(float) * mm, cudaMemcpyDeviceToDevice, st));
        TSVM_TRY(ensure_planes(km, st));
        TSVM_LAUNCH(stage_rows_dense_kernel, mm, 256, 0, st, T_dev + (size_t) r0 * ldt, ldt, km->d, km->d, mm,
                    row_dst(km));
        TSVM_TRY(rows_common(km, mm, out_dev + (size_t) r0 * ld_out, ld_out, st));
    }
    return TSVM_OK;
}

tsvm_status tsvm_km_rows_by_instances_csr(tsvm_km *km, const float *tval_dev, const int *trow_ptr_dev,
                                          const int *tcol_dev, int m, long long tnnz, float *out_dev,
                                          long long ld_out, void *stream) {
    (void) tnnz;
    TSVM_REQUIRE(km && trow_ptr_dev && out_dev && m > 0 && ld_out >= km->n, "rows_by_instances_csr: bad arguments");
    cudaStream_t st = (cudaStream_t) stream;
    const int chunk = km->dense ? 4096 : 1024;
    for (int r0 = 0; r0 < m; r0 += chunk) {
        const int mm = min(chunk, m - r0);
        const int *rp = trow_ptr_dev + r0;     // row_ptr entries stay absolute offsets into tval/tcol
        float *o = out_dev + (size_t) r0 * ld_out;
        if (km->dense) {
            TSVM_TRY(km_stage_instances_csr(km, tval_dev, rp, tcol_dev, mm, st));
            TSVM_TRY(rows_common(km, mm, o, ld_out, st));
        } else {
            TSVM_TRY(ensure_scratch(km, mm));
            TSVM_LAUNCH(self_dot_seq_csr_kernel, ceil_div(mm, 128), 128, 0, st, tval_dev, rp, mm, km->sd_rows);
            TSVM_LAUNCH(scatter_csr_to_wt_kernel, mm, 128, 0, st, tval_dev, rp, tcol_dev, (const int *) nullptr, mm,
                        km->d, km->wt_ld, km->WT, (const float *) nullptr, (float *) nullptr, false, (const int *) nullptr);
            TSVM_TRY(rows_common(km, mm, o, ld_out, st));
            TSVM_LAUNCH(scatter_csr_to_wt_kernel, mm, 128, 0, st, tval_dev, rp, tcol_dev, (const int *) nullptr, mm,
                        km->d, km->wt_ld, km->WT, (const float *) nullptr, (float *) nullptr, true, (const int *) nullptr);
        }
    }
    return TSVM_OK;
}

}  // extern "C"
