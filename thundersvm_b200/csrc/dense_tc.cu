// Dense kernel rows on the 5th-generation tensor cores (sm_100a):
//
//     out[i][j] = kfn( sum_k W[i][k] * X[j][k] ),   i < m requested rows, j < n instances
//
// as an error-compensated 3xTF32 contraction. Both operands are stored split into two TF32
// planes (x = hi + lo); every k-step issues three tcgen05.mma (lo*hi, hi*lo, hi*hi) into an
// FP32 accumulator in tensor memory. Operand tiles travel HBM/L2 -> shared memory by TMA
// (128-byte swizzle, zero fill outside the matrices).
//
// The tensor core adds into its accumulator with truncation (measured: about half an ulp of the
// accumulator lost per MMA, always towards zero), which on long same-sign sums is far outside
// the 1e-5 bound on kernel values. Tensor memory therefore only ever holds the partial sum of
// ONE 32-wide k slab: the two 256-column accumulators alternate slab by slab, and the epilogue
// warps move every finished slab into FP32 registers (tcgen05.ld + round-to-nearest adds on the
// CUDA cores) while the tensor core works on the next slab. The kernel function (RBF /
// polynomial / sigmoid / linear, with the self-dot norms) is applied to the register sums
// before the only store to HBM.
//
// Replaces the reference's cublasSgemm + separate RBF pass
// (src/thundersvm/kernel/kernelmatrix_kernel.cu:311-330, 58-67; kernelmatrix.cpp:318-343).
//
// CTA layout (320 threads, one CTA per SM, persistent over tiles):
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : allocates tensor memory, issues the MMAs (one elected lane)
//   warps 2..9  : slab promotion + epilogue; warp w owns tensor-memory lanes 32*(w%4) .. +31 and
//                 columns 128*((w-2)/4) .. +127 (128 FP32 sums per thread)
// Tile: 128 instances (MMA M, tensor-memory lanes) x 256 requested rows (MMA N, columns).
// Every wait is bounded; on expiry the kernel records a status word and winds down.
#include "tc_common.cuh"

namespace tsvm {

namespace tc {
constexpr int BM = 128, BN = 256, BK = 32, STAGES = 2, UMMA_K = 8;
constexpr uint32_t A_BYTES = BM * BK * 4;          // 16 KB per plane
constexpr uint32_t B_BYTES = BN * BK * 4;          // 32 KB per plane
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;   // 96 KB
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr int THREADS = 320, EPI_WARPS = 8, COLS_PER_THREAD = 128;
constexpr uint32_t TMEM_COLS = 512;
// tcgen05 instruction descriptor: D=F32, A=B=TF32, both K-major, N=256, M=128
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t) (BN >> 3) << 17) |
                           ((uint32_t) (BM >> 4) << 24);
}  // namespace tc

template <int EPI>
__global__ void __launch_bounds__(tc::THREADS, 1)
dense_rows_tc_kernel(const __grid_constant__ CUtensorMap map_xhi, const __grid_constant__ CUtensorMap map_xlo,
                     const __grid_constant__ CUtensorMap map_whi, const __grid_constant__ CUtensorMap map_wlo,
                     int n, int m, int d_pad, const float *__restrict__ sd, const float *__restrict__ sd_rows,
                     KernelFn fn, float *__restrict__ out, long long ld_out, int *__restrict__ status) {
    using namespace tc;
    extern __shared__ uint8_t smem_raw[];
    // operand ring, 1024-byte aligned (swizzle atom = 8 rows x 128 B)
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring_ptr + STAGES * STAGE_BYTES);
    const uint32_t full_bar = smem_u32(bars), empty_bar = full_bar + 8 * STAGES;
    const uint32_t tfull_bar = empty_bar + 8 * STAGES, tempty_bar = tfull_bar + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (n + BM - 1) / BM, n_blocks = (m + BN - 1) / BN, k_blocks = (d_pad + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar + 8 * a, 1); mbar_init(tempty_bar + 8 * a, EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x)
                for (int nb = 0; nb < n_blocks && ok; ++nb)
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                        const uint32_t fb = full_bar + 8 * stage, base = ring + stage * STAGE_BYTES;
                        mbar_expect_tx(fb, STAGE_BYTES);
                        tma_load_2d(base, &map_xhi, fb, kb * BK, mt * BM);
                        tma_load_2d(base + A_BYTES, &map_xlo, fb, kb * BK, mt * BM);
                        tma_load_2d(base + 2 * A_BYTES, &map_whi, fb, kb * BK, nb * BN);
                        tma_load_2d(base + 2 * A_BYTES + B_BYTES, &map_wlo, fb, kb * BK, nb * BN);
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: one k slab per tensor-memory accumulator ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x)
                for (int nb = 0; nb < n_blocks && ok; ++nb)
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, 2)) { ok = false; break; }
                        if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, 3)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t d_tmem = tmem_base + acc * BN;
                        const uint32_t base = ring + stage * STAGE_BYTES;
                        // the two small cross terms first, while the accumulator is still tiny
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint32_t koff = k * UMMA_K * 4;
                            umma_tf32(d_tmem, smem_desc_sw128(base + A_BYTES + koff),
                                      smem_desc_sw128(base + 2 * A_BYTES + koff), IDESC, k != 0);
                            umma_tf32(d_tmem, smem_desc_sw128(base + koff),
                                      smem_desc_sw128(base + 2 * A_BYTES + B_BYTES + koff), IDESC, 1);
                        }
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint32_t koff = k * UMMA_K * 4;
                            umma_tf32(d_tmem, smem_desc_sw128(base + koff), smem_desc_sw128(base + 2 * A_BYTES + koff), IDESC, 1);
                        }
                        umma_commit(empty_bar + 8 * stage);      // smem stage reusable once these MMAs retire
                        umma_commit(tfull_bar + 8 * acc);        // slab sum complete in tensor memory
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                    }
        }
    } else {
        // ---------------- slab promotion + epilogue ----------------
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x) {
            const int j = mt * BM + quarter * 32 + lane;
            const float sdj = j < n ? sd[j] : 0.0f;
            for (int nb = 0; nb < n_blocks && ok; ++nb) {
                float sum[COLS_PER_THREAD];
#pragma unroll
                for (int c = 0; c < COLS_PER_THREAD; ++c) sum[c] = 0.0f;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, 4)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((uint32_t) (quarter * 32) << 16) + acc * BN + half * COLS_PER_THREAD;
#pragma unroll
                    for (int c0 = 0; c0 < COLS_PER_THREAD; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(taddr + c0, v);
#pragma unroll
                        for (int c = 0; c < 32; ++c) sum[c0 + c] += __uint_as_float(v[c]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                }
                if (!ok) break;
                if (j < n) {
                    const int i0 = nb * BN + half * COLS_PER_THREAD;
#pragma unroll
                    for (int c = 0; c < COLS_PER_THREAD; ++c) {
                        const int i = i0 + c;
                        if (i < m) out[(size_t) i * ld_out + j] = epilogue_value<EPI>(fn, sum[c], __ldg(sd_rows + i), sdj);
                    }
                }
            }
        }
    }

    // wind-down: on the error path give in-flight bulk copies time to land before the shared
    // memory and tensor memory are released.
    if (*abort_flag) {
        const long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ll) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    if (threadIdx.x == 0 && *abort_flag) atomicMax(status, *abort_flag);
}

// ---- host ------------------------------------------------------------------------------------

typedef CUresult (*encode_fn_t)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_fn_t get_encode() {
    static encode_fn_t fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (encode_fn_t) p;
    }
    return fn;
}

// rows x row_len matrix of 32-bit words (or FP16 halves) with row stride ld elements; box = one 128-byte
// swizzle row (32 words / 64 halves) x box_rows rows.
tsvm_status make_map(CUtensorMap *map, const void *ptr, int rows, int row_len, long long ld, int box_rows, bool f16) {
    encode_fn_t enc = get_encode();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return TSVM_ERR_CUDA; }
    const size_t esz = f16 ? 2 : 4;
    cuuint64_t dims[2] = {(cuuint64_t) row_len, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) ld * esz};
    cuuint32_t box[2] = {(cuuint32_t) (128 / esz), (cuuint32_t) box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *) ptr, dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int) r); return TSVM_ERR_CUDA; }
    return TSVM_OK;
}

// Whi/Wlo (m x d_pad) and sd_rows are staged in the handle's scratch by the caller.
tsvm_status launch_dense_tc2(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st);   // dense_tc2.cu

tsvm_status launch_dense_tc(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st) {
    // engine 2 forces the single-CTA tiles; otherwise CTA pairs (also for one tile: the second CTA idles)
    if (km->engine != 2) return launch_dense_tc2(km, m, out, ld_out, st);
    TSVM_REQUIRE(km->plane_kind == 1, "single-CTA tensor engine needs TF32 planes");
    CUtensorMap mxh, mxl, mwh, mwl;
    TSVM_TRY(make_map(&mxh, km->Xhi, km->n, km->d_pad, km->d_pad, tc::BM, false));
    TSVM_TRY(make_map(&mxl, km->Xlo, km->n, km->d_pad, km->d_pad, tc::BM, false));
    TSVM_TRY(make_map(&mwh, km->Whi, m, km->d_pad, km->d_pad, tc::BN, false));
    TSVM_TRY(make_map(&mwl, km->Wlo, m, km->d_pad, km->d_pad, tc::BN, false));
    int dev = 0, sms = 0;
    TSVM_CUDA(cudaGetDevice(&dev));
    TSVM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    TSVM_ONCE_PER_DEVICE({
        TSVM_CUDA(cudaFuncSetAttribute(dense_rows_tc_kernel<EPI_RBF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int) tc::SMEM_BYTES));
        TSVM_CUDA(cudaFuncSetAttribute(dense_rows_tc_kernel<EPI_LINEAR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int) tc::SMEM_BYTES));
        TSVM_CUDA(cudaFuncSetAttribute(dense_rows_tc_kernel<EPI_GENERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int) tc::SMEM_BYTES));
    });
    const int m_tiles = ceil_div(km->n, tc::BM);
    const int grid = m_tiles < sms ? m_tiles : sms;
#define TC_LAUNCH(E)                                                                                              \
    TSVM_LAUNCH(dense_rows_tc_kernel<E>, grid, tc::THREADS, tc::SMEM_BYTES, st, mxh, mxl, mwh, mwl, km->n, m,     \
                km->d_pad, km->self_dot, km->sd_rows, km->fn, out, ld_out, km->status_dev)
    switch (epilogue_kind(km->fn)) {
        case EPI_RBF: TC_LAUNCH(EPI_RBF); break;
        case EPI_LINEAR: TC_LAUNCH(EPI_LINEAR); break;
        default: TC_LAUNCH(EPI_GENERIC); break;
    }
#undef TC_LAUNCH
    return TSVM_OK;
}

}  // namespace tsvm
