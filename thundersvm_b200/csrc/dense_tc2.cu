// Dense kernel rows on tcgen05 with CTA pairs (cta_group::2).
//
// Same contraction, same 3xTF32 scheme and same per-slab FP32 promotion as dense_tc.cu, but two
// CTAs on neighbouring SMs work as one: the pair owns a 256-instance x 256-requested-row tile, each
// CTA holds the TF32 planes of ITS 128 instances and of ITS 128 requested rows (half of the B
// operand), and one thread of the leader CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads
// both CTAs' shared memory and writes both CTAs' tensor memory. Per CTA a k slab is then 64 KB
// instead of 96 KB for the same tensor-core time, and three of them fit the ring instead of two - the
// single-CTA engine was bound by the latency of its one slab in flight, not by any bandwidth.
//
// Roles per CTA (384 threads = 3 warpgroups): warp 0 TMA producer for this CTA's operand halves
// (transaction bytes are reported to the leader's "full" barrier), warp 1 tensor-memory allocation (both
// CTAs) and MMA issue (leader only), warps 2..3 idle, warps 4..11 slab promotion + epilogue on this CTA's 128
// instances. Warpgroup 0 hands registers to the other two (setmaxnreg): the epilogue keeps 128 sums per
// thread live, and with the 168 registers a 384-thread CTA is compiled for it spilled a few loop-invariant
// values - their reloads from local memory (the L1 is tiny next to 222 KB of shared memory) cost 9 % of
// the kernel.
// Barriers: full[s] (leader; both CTAs' TMA bytes), empty[s] (per CTA; MMAs that read the stage have
// retired), tfull[a] (per CTA; slab sum complete), tempty[a] (leader; 16 epilogue warps drained it).
// Cross-CTA signalling uses mbarrier arrives on shared::cluster addresses and one tcgen05.commit per
// destination CTA; every load is addressed to one CTA's shared memory only. Every mbarrier wait is bounded.
#include "tc_common.cuh"

#ifndef TSVM_PROMO
#define TSVM_PROMO 2
#endif

namespace tsvm {

namespace tc2 {
// A k slab is one 128-byte swizzle row per matrix row: 32 TF32 words or 64 FP16 halves, four MMA k-steps
// of 32 bytes either way.
constexpr int BM = 128, BN = 256, BN_HALF = 128, STAGES = 3, K_STEPS = 4;
constexpr uint32_t A_BYTES = BM * 128;               // 16 KB per plane (this CTA's instances)
constexpr uint32_t B_BYTES = BN_HALF * 128;          // 16 KB per plane (this CTA's half of the requested rows)
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;   // 64 KB per CTA
// Warpgroup 0 holds the TMA producer (warp 0), the MMA issuer (warp 1) and two idle warps and gives most of its
// registers back; the other warpgroups are the promotion / epilogue warps and take them. Default: 8 epilogue
// warps (two per tensor-memory lane quarter, 128 columns = 128 sums per thread; a 384-thread CTA is compiled
// for 168 registers: 128 * 56 + 256 * 224). TSVM_EPI_WARPS = 16 (four per quarter, 64 sums per thread, 640
// threads) builds and passes the same tests; measured on the 400,000 x 2,000 launch it changes nothing
// (1.90 ms against 1.88 ms) - the kernel waits for the tensor pipe, not for its epilogue.
#ifndef TSVM_EPI_WARPS
#define TSVM_EPI_WARPS 8
#endif
constexpr int EPI_WARPS = TSVM_EPI_WARPS, EPI_WARP0 = 4, THREADS = 32 * (EPI_WARP0 + EPI_WARPS);
constexpr int COLS_PER_THREAD = BN / (EPI_WARPS / 4);
// Registers can only move inside the CTA: what the epilogue warps take (setmaxnreg.inc blocks until it is there)
// must have been given back by the control warps, counted from the per-thread figure the kernel is compiled and
// launched with (168 for 384 threads, 96 for 640: the largest multiples of 8 that fit 65,536 registers).
constexpr int REGS_LAUNCH = EPI_WARPS == 8 ? 168 : 96;
constexpr int REGS_CONTROL = EPI_WARPS == 8 ? 56 : 32, REGS_EPILOGUE = EPI_WARPS == 8 ? 224 : 112;
static_assert(EPI_WARPS == 8 || EPI_WARPS == 16, "two or four epilogue warps per tensor-memory lane quarter");
static_assert(128 * REGS_CONTROL + 32 * EPI_WARPS * REGS_EPILOGUE <= THREADS * REGS_LAUNCH,
              "the epilogue warps would wait for registers that nobody releases");
static_assert(THREADS * REGS_LAUNCH <= 65536, "register file of an SM");
// epilogue staging (see the epilogue): EPI_CHUNK sums of each epilogue thread (eight chunks per thread), and per
// warp the self dots and 1/scale of its requested rows
constexpr int EPI_CHUNK = COLS_PER_THREAD / 8;
constexpr uint32_t EPI_STAGE_BYTES = EPI_CHUNK * EPI_WARPS * 32 * 4;
constexpr uint32_t EPI_CONST_BYTES = EPI_WARPS * 2 * COLS_PER_THREAD * 4;
// prediction form: up to PRED_NC_SMEM coefficients of every epilogue thread's own instance (thread-private columns)
constexpr int PRED_NC_SMEM = EPI_WARPS == 8 ? 9 : 4;
constexpr uint32_t PRED_BYTES = PRED_NC_SMEM * EPI_WARPS * 32 * 4;
// kernel-row form: output row (slot of the caller's row buffer) of every requested row, per epilogue warp
constexpr uint32_t SLOT_BYTES = EPI_WARPS * COLS_PER_THREAD * 4;
constexpr uint32_t SMEM_BASE = STAGES * STAGE_BYTES + 1024 + 256 + EPI_STAGE_BYTES + EPI_CONST_BYTES;
constexpr uint32_t SMEM_BYTES = SMEM_BASE + SLOT_BYTES;
constexpr uint32_t SMEM_BYTES_PREDICT = SMEM_BASE + PRED_BYTES;
static_assert(SMEM_BYTES <= 227 * 1024, "kernel-row form does not fit the shared memory of an SM");
static_assert(SMEM_BYTES_PREDICT <= 227 * 1024, "prediction form does not fit the shared memory of an SM");
constexpr uint32_t TMEM_COLS = 512;
// D=F32, K-major, M=256 (two CTAs x 128); A=B=TF32 (format 2) or F16 (format 0)
// (the N field, bits 17.., is added per row block: a block's last rows may need fewer than 256 columns)
constexpr uint32_t IDESC_SHAPE = (1u << 4) | ((uint32_t) (256 >> 4) << 24);
constexpr uint32_t IDESC_TF32 = IDESC_SHAPE | (2u << 7) | (2u << 10);
constexpr uint32_t IDESC_F16 = IDESC_SHAPE;
}  // namespace tc2

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: data lands in this CTA's shared memory, the bytes are counted on the
// barrier at the given shared::cluster address (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
// idesc_n: the instruction descriptor's N field ((N >> 3) << 17); a row block with few requested rows left
// issues narrower MMAs
template <bool F16>
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate,
                                          uint32_t idesc_n) {
    if constexpr (F16)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(tc2::IDESC_F16 | idesc_n), "r"(accumulate) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(tc2::IDESC_TF32 | idesc_n), "r"(accumulate) : "memory");
}
// arrives on the barrier at a shared::cluster address once all MMAs issued so far have retired
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

// sums [CH * EPI_CHUNK, (CH + 1) * EPI_CHUNK) of the thread -> its private column of the staging block
template <int CH>
__device__ __forceinline__ void stage_chunk(const float (&sum)[tc2::COLS_PER_THREAD], float *priv) {
    static_assert(tc2::COLS_PER_THREAD / tc2::EPI_CHUNK == 8, "the epilogue's switch lists eight chunks");
#pragma unroll
    for (int c = 0; c < tc2::EPI_CHUNK; ++c) priv[c * (tc2::EPI_WARPS * 32)] = sum[CH * tc2::EPI_CHUNK + c];
}

// Prediction form of the kernel (PREDICT = true): the instances are the support vectors, the requested rows
// the test rows, and instead of writing the kernel values the epilogue multiplies them by the support
// vectors' coefficients and adds the sums to the decision values - svm_kernel::sum_kernel_values
// (src/thundersvm/kernel/kernelmatrix_kernel.cu:69-97) folded into the contraction, so that the
// test x SV kernel block never reaches HBM.
struct PredictArgs {
    const double *coef;        // (n_classes - 1) x n_sv, the model's layout (include/thundersvm/model/svmmodel.h:155-164)
    const int *sv_class;       // class of every support vector [n_sv]
    double *dec;               // [m][n_pairs], preset to -rho; this launch adds its sums
    int n_classes, n_pairs;
};

// Optional indirections of the kernel-row form, both read on the device so that a caller can decide them
// without a host round trip: the number of requested rows actually wanted (at most the m the launch was
// sized for) and, per requested row, the row of `out` it is written to.
struct RowsExtra {
    const int *m_dev;
    const int *row_slot;
};

__device__ __forceinline__ int pair_index(int n_classes, int i, int j) {      // i < j, pairs ordered (0,1),(0,2),...
    return i * (2 * n_classes - i - 1) / 2 + (j - i - 1);
}

// Columns (requested rows) of row block nb that the MMAs cover: all 256, or the rows left rounded up to 32
__device__ __forceinline__ int block_columns(int m, int nb) {
    const int left = m - nb * tc2::BN;
    return left >= tc2::BN ? tc2::BN : ((left + 31) & ~31);
}

template <int EPI, bool F16, bool PREDICT>
__global__ void __launch_bounds__(tc2::THREADS, 1)
dense_rows_tc2_kernel(const __grid_constant__ CUtensorMap map_xhi, const __grid_constant__ CUtensorMap map_xlo,
                      const __grid_constant__ CUtensorMap map_whi, const __grid_constant__ CUtensorMap map_wlo,
                      int n, int m_launch, int row_len, const float *__restrict__ sd, const float *__restrict__ sd_rows,
                      const float *__restrict__ x_unscale, const float *__restrict__ w_unscale,
                      KernelFn fn, float *__restrict__ out, long long ld_out, int *__restrict__ status,
                      const PredictArgs pa, const RowsExtra ex) {
    using namespace tc2;
    // the same value in every thread of the grid: the launch's m, or the smaller count found on the device
    const int m = ex.m_dev ? min(m_launch, max(*ex.m_dev, 0)) : m_launch;
    constexpr int BK = F16 ? 64 : 32;          // elements per k slab
    constexpr int PROMO = F16 ? TSVM_PROMO : 1;   // k slabs summed in tensor memory before the FP32 promotion
    extern __shared__ uint8_t smem_raw[];
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring_ptr + STAGES * STAGE_BYTES);
    const uint32_t full_bar = smem_u32(bars), empty_bar = full_bar + 8 * STAGES;
    const uint32_t tfull_bar = empty_bar + 8 * STAGES, tempty_bar = tfull_bar + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int pair_tiles = (n + 2 * BM - 1) / (2 * BM), n_blocks = (m + BN - 1) / BN, k_blocks = (row_len + BK - 1) / BK;
    // Work items are (pair tile, row block) with the row block fastest, so neighbouring clusters stream the
    // same instance slabs at the same time and the second reader finds them in L2.
    const int n_items = pair_tiles * n_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + 8 * s, 1); mbar_init(empty_bar + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar + 8 * a, 1); mbar_init(tempty_bar + 8 * a, 2 * EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();           // both CTAs' barriers are initialised before any remote arrive / TMA
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < EPI_WARP0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_CONTROL));
    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int item = cluster_id; item < n_items && ok; item += n_clusters) {
                    const int pt = item / n_blocks, nb = item - pt * n_blocks;
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                        const uint32_t base = ring + stage * STAGE_BYTES;
                        const uint32_t leader_full = mapa_u32(full_bar + 8 * stage, 0);
                        if (rank == 0) mbar_expect_tx(full_bar + 8 * stage, 2 * STAGE_BYTES);
                        // this CTA's half of the block's requested rows (a narrow last block has narrow halves)
                        const int xrow = pt * 2 * BM + (int) rank * BM, wrow = nb * BN + (int) rank * (block_columns(m, nb) >> 1);
                        tma_load_2d_pair(base, &map_xhi, leader_full, kb * BK, xrow);
                        tma_load_2d_pair(base + A_BYTES, &map_xlo, leader_full, kb * BK, xrow);
                        tma_load_2d_pair(base + 2 * A_BYTES, &map_whi, leader_full, kb * BK, wrow);
                        tma_load_2d_pair(base + 2 * A_BYTES + B_BYTES, &map_wlo, leader_full, kb * BK, wrow);
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int item = cluster_id; item < n_items && ok; item += n_clusters) {
                    const uint32_t idesc_n = (uint32_t) (block_columns(m, item % n_blocks) >> 3) << 17;
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        const bool unit_start = kb % PROMO == 0, unit_end = kb % PROMO == PROMO - 1 || kb == k_blocks - 1;
                        if (unit_start && !mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, 2)) { ok = false; break; }
                        if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, 3)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t d_tmem = tmem_base + acc * BN;
                        const uint32_t base = ring + stage * STAGE_BYTES;
#pragma unroll
                        for (int k = 0; k < K_STEPS; ++k) {
                            const uint32_t koff = k * 32;
                            umma_pair<F16>(d_tmem, smem_desc_sw128(base + A_BYTES + koff),
                                           smem_desc_sw128(base + 2 * A_BYTES + koff), k != 0 || !unit_start, idesc_n);
                            umma_pair<F16>(d_tmem, smem_desc_sw128(base + koff),
                                           smem_desc_sw128(base + 2 * A_BYTES + B_BYTES + koff), 1, idesc_n);
                        }
#pragma unroll
                        for (int k = 0; k < K_STEPS; ++k) {
                            const uint32_t koff = k * 32;
                            umma_pair<F16>(d_tmem, smem_desc_sw128(base + koff), smem_desc_sw128(base + 2 * A_BYTES + koff), 1, idesc_n);
                        }
                        // stage free / slab complete, signalled in both CTAs
                        umma_commit_pair(mapa_u32(empty_bar + 8 * stage, 0));
                        umma_commit_pair(mapa_u32(empty_bar + 8 * stage, 1));
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                        if (unit_end) {
                            umma_commit_pair(mapa_u32(tfull_bar + 8 * acc, 0));
                            umma_commit_pair(mapa_u32(tfull_bar + 8 * acc, 1));
                            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                        }
                    }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_EPILOGUE));
        // ---------------- slab promotion + epilogue (both CTAs, own 128 instances) ----------------
        const int quarter = warp & 3, half = (warp - EPI_WARP0) >> 2;
        float *priv = reinterpret_cast<float *>(ring_ptr + STAGES * STAGE_BYTES + 256) + (warp - EPI_WARP0) * 32 + lane;
        float *rowc = reinterpret_cast<float *>(ring_ptr + STAGES * STAGE_BYTES + 256 + EPI_STAGE_BYTES) +
                      (warp - EPI_WARP0) * 2 * COLS_PER_THREAD;
        int *slotc = reinterpret_cast<int *>(ring_ptr + STAGES * STAGE_BYTES + 256 + EPI_STAGE_BYTES + EPI_CONST_BYTES) +
                     (warp - EPI_WARP0) * COLS_PER_THREAD;
        // prediction form: the coefficients of the thread's own instance, one thread-private column
        float *coef_priv = reinterpret_cast<float *>(ring_ptr + STAGES * STAGE_BYTES + 256 + EPI_STAGE_BYTES + EPI_CONST_BYTES) +
                           (warp - EPI_WARP0) * 32 + lane;
        const int nc = PREDICT ? pa.n_classes - 1 : 0;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (int item = cluster_id; item < n_items && ok; item += n_clusters) {
            const int pt = item / n_blocks, nb = item - pt * n_blocks;
            const int j = pt * 2 * BM + (int) rank * BM + quarter * 32 + lane;
            const float sdj = j < n ? sd[j] : 0.0f;
            const float uxj = (F16 && j < n) ? x_unscale[j] : 1.0f;
            const int n_cols = block_columns(m, nb);
            int cls_own = 0, cls_lo = 0, cls_hi = -1;
            float coef_one = 0.0f;
            if constexpr (PREDICT) {
                // class and coefficients of the thread's own instance (a lane beyond the last instance takes the
                // last one's class; its kernel values are forced to zero)
                cls_own = pa.sv_class[j < n ? j : n - 1];
                if (nc == 1) coef_one = j < n ? (float) pa.coef[j] : 0.0f;
                else if (nc <= PRED_NC_SMEM)
                    for (int cr = 0; cr < nc; ++cr)
                        coef_priv[cr * (EPI_WARPS * 32)] = j < n ? (float) pa.coef[(size_t) cr * n + j] : 0.0f;
            }
            {
                // Self dot and 1/scale of this warp's 128 requested rows go to shared memory by asynchronous
                // copies while the k loop runs: with nearly all of the SM's memory configured as shared, the
                // L1 left over does not keep them across the epilogue's stores.
                const int i0 = nb * BN + half * COLS_PER_THREAD;
#pragma unroll
                for (int c = lane; c < COLS_PER_THREAD; c += 32) {
                    if (i0 + c < m) {
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(rowc + c)), "l"(sd_rows + i0 + c) : "memory");
                        if constexpr (F16)
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(rowc + COLS_PER_THREAD + c)), "l"(w_unscale + i0 + c) : "memory");
                        if constexpr (!PREDICT)
                            if (ex.row_slot)
                                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(slotc + c)), "l"(ex.row_slot + i0 + c) : "memory");
                    }
                }
                float sum[COLS_PER_THREAD];
#pragma unroll
                for (int c = 0; c < COLS_PER_THREAD; ++c) sum[c] = 0.0f;
                for (int unit = 0; unit < (k_blocks + PROMO - 1) / PROMO; ++unit) {
                    if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, 4)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((uint32_t) (quarter * 32) << 16) + acc * BN + half * COLS_PER_THREAD;
#pragma unroll
                    for (int c0 = 0; c0 < COLS_PER_THREAD; c0 += 32) {
                        if (half * COLS_PER_THREAD + c0 >= n_cols) break;      // columns the narrow MMAs did not write
                        uint32_t v[32];
                        tmem_ld32(taddr + c0, v);
#pragma unroll
                        for (int c = 0; c < 32; ++c) sum[c0 + c] += __uint_as_float(v[c]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar + 8 * acc, 0));
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                }
                if (!ok) break;
                // The sums live in registers, so a loop over them has to be fully unrolled; with the kernel
                // function in its body that is 128 copies of it, and the instruction fetch of such an
                // epilogue cost several times its arithmetic. Instead the sums pass 32 at a time through a
                // thread-private column of shared memory (no synchronisation: every thread reads back only
                // what it wrote), 16 at a time, and a short rolled loop applies the kernel function and stores.
                asm volatile("cp.async.wait_all;" ::: "memory");
                __syncwarp();
                // prediction form, RBF: K = 2^(A_i + B_j + S_i * dot) with per-test-row constants A_i, S_i (they
                // replace the row's self dot and 1/scale in rowc) and the own instance's B_j: four instructions
                // per kernel value. The exponent is formed in FP32 without the residual correction the stored
                // kernel rows use (relative error up to |exponent| * 2^-23), which decision values do not need.
                float pred_b = 0.0f;
                if constexpr (PREDICT && EPI == EPI_RBF) {
                    constexpr float LOG2E = 1.4426950408889634f;
                    cls_lo = __reduce_min_sync(0xffffffffu, cls_own);
                    cls_hi = __reduce_max_sync(0xffffffffu, cls_own);
                    pred_b = -fn.gamma * LOG2E * sdj;
#pragma unroll
                    for (int c = lane; c < COLS_PER_THREAD; c += 32) {
                        const float sd_i = rowc[c];
                        const float uw_i = F16 ? rowc[COLS_PER_THREAD + c] : 1.0f;
                        rowc[c] = -fn.gamma * LOG2E * sd_i;
                        rowc[COLS_PER_THREAD + c] = 2.0f * fn.gamma * LOG2E * uw_i;
                    }
                    __syncwarp();
                } else if constexpr (PREDICT) {
                    cls_lo = __reduce_min_sync(0xffffffffu, cls_own);
                    cls_hi = __reduce_max_sync(0xffffffffu, cls_own);
                }
#pragma unroll 1
                for (int ch = 0; ch < COLS_PER_THREAD / EPI_CHUNK; ++ch) {
                    if (half * COLS_PER_THREAD + ch * EPI_CHUNK >= n_cols) break;
                    switch (ch) {           // register indices must be constants: one short case per chunk
                        case 0: stage_chunk<0>(sum, priv); break;
                        case 1: stage_chunk<1>(sum, priv); break;
                        case 2: stage_chunk<2>(sum, priv); break;
                        case 3: stage_chunk<3>(sum, priv); break;
                        case 4: stage_chunk<4>(sum, priv); break;
                        case 5: stage_chunk<5>(sum, priv); break;
                        case 6: stage_chunk<6>(sum, priv); break;
                        default: stage_chunk<7>(sum, priv); break;
                    }
                    const int cbase = ch * EPI_CHUNK;
                    if constexpr (!PREDICT) {
                        if (j < n) {
                            const int lim = m - (i0 + cbase) < EPI_CHUNK ? m - (i0 + cbase) : EPI_CHUNK;
                            if (!ex.row_slot) {
                                float *o = out + (size_t) (i0 + cbase) * ld_out + j;
#pragma unroll 8
                                for (int c = 0; c < lim; ++c) {
                                    float dot = priv[c * (EPI_WARPS * 32)];
                                    if constexpr (F16) dot = dot * uxj * rowc[COLS_PER_THREAD + cbase + c];
                                    o[(size_t) c * ld_out] = epilogue_value<EPI>(fn, dot, rowc[cbase + c], sdj);
                                }
                            } else {
#pragma unroll 8
                                for (int c = 0; c < lim; ++c) {
                                    float dot = priv[c * (EPI_WARPS * 32)];
                                    if constexpr (F16) dot = dot * uxj * rowc[COLS_PER_THREAD + cbase + c];
                                    out[(size_t) slotc[cbase + c] * ld_out + j] = epilogue_value<EPI>(fn, dot, rowc[cbase + c], sdj);
                                }
                            }
                        }
                    } else {
                        // Kernel values of the own instance for the chunk's 16 test rows, times the instance's
                        // coefficient; then the 32 lanes' products are added column by column with a butterfly
                        // that halves the number of live columns per step (16 -> 8 -> 4 -> 2 -> 1 values per
                        // lane, 31 shuffles for 16 columns), and one lane of every pair adds the warp's sum of
                        // its column to the decision value. No exchange between warps: every warp adds the sums
                        // of its own 32 instances.
                        float kv[EPI_CHUNK];
                        if constexpr (EPI == EPI_RBF) {
                            float a_i[EPI_CHUNK], s_i[EPI_CHUNK];
#pragma unroll
                            for (int c4 = 0; c4 < EPI_CHUNK; c4 += 4) {
                                const float4 av = *reinterpret_cast<const float4 *>(rowc + cbase + c4);
                                const float4 sv = *reinterpret_cast<const float4 *>(rowc + COLS_PER_THREAD + cbase + c4);
                                a_i[c4] = av.x; a_i[c4 + 1] = av.y; a_i[c4 + 2] = av.z; a_i[c4 + 3] = av.w;
                                s_i[c4] = sv.x; s_i[c4 + 1] = sv.y; s_i[c4 + 2] = sv.z; s_i[c4 + 3] = sv.w;
                            }
#pragma unroll
                            for (int c = 0; c < EPI_CHUNK; ++c) {
                                float dot = priv[c * (EPI_WARPS * 32)];
                                if constexpr (F16) dot *= uxj;
                                const float arg = fmaf(dot, s_i[c], a_i[c]) + pred_b;
                                float e;
                                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(arg));
                                kv[c] = j < n ? e : 0.0f;
                            }
                        } else {
#pragma unroll
                            for (int c = 0; c < EPI_CHUNK; ++c) {
                                float dot = priv[c * (EPI_WARPS * 32)];
                                if constexpr (F16) dot = dot * uxj * rowc[COLS_PER_THREAD + cbase + c];
                                kv[c] = j < n ? epilogue_value<EPI>(fn, dot, rowc[cbase + c], sdj) : 0.0f;
                            }
                        }
                        // column of the chunk this lane ends up with: lane bit 16 >> s selects the upper half of step s
                        int col = 0;
#pragma unroll
                        for (int st = 0, hn = EPI_CHUNK / 2; hn >= 1; ++st, hn >>= 1) col += ((lane >> (4 - st)) & 1) * hn;
                        constexpr int REST = 32 / EPI_CHUNK;             // lanes that hold the same column afterwards
                        const int r = i0 + cbase + col;
                        for (int cl = cls_lo; cl <= cls_hi; ++cl)
                            for (int cr = 0; cr < nc; ++cr) {
                                float cf;
                                if (nc == 1) cf = coef_one;
                                else if (nc <= PRED_NC_SMEM) cf = coef_priv[cr * (EPI_WARPS * 32)];
                                else cf = j < n ? (float) pa.coef[(size_t) cr * n + j] : 0.0f;
                                if (cls_own != cl) cf = 0.0f;
                                float w[EPI_CHUNK];
#pragma unroll
                                for (int c = 0; c < EPI_CHUNK; ++c) w[c] = cf * kv[c];
#pragma unroll
                                for (int st = 0, half_n = EPI_CHUNK / 2; half_n >= 1; ++st, half_n >>= 1) {
                                    const int bit = 16 >> st;                          // lane bit 4, 3, 2, ...
                                    const bool upper = (lane & bit) != 0;
#pragma unroll
                                    for (int c = 0; c < half_n; ++c) {
                                        const float send = upper ? w[c] : w[c + half_n];
                                        const float keep = upper ? w[c + half_n] : w[c];
                                        w[c] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                                    }
                                }
                                float total = w[0];
#pragma unroll
                                for (int o = REST >> 1; o >= 1; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                                if ((lane & (REST - 1)) == 0 && r < m && total != 0.0f) {
                                    const int other = cr < cl ? cr : cr + 1;
                                    const int k = other > cl ? pair_index(pa.n_classes, cl, other)
                                                             : pair_index(pa.n_classes, other, cl);
                                    atomicAdd(pa.dec + (size_t) r * pa.n_pairs + k, (double) total);
                                }
                            }
                    }
                }
                __syncwarp();          // the next item's copies overwrite rowc
            }
        }
    }

    if (*abort_flag) {
        const long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ll) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();           // neither CTA leaves while its partner may still signal it or read its memory
    tc_fence_after();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    if (threadIdx.x == 0 && *abort_flag) atomicMax(status, *abort_flag);
}

tsvm_status make_map(CUtensorMap *map, const void *ptr, int rows, int row_len, long long ld, int box_rows,
                     bool f16);   // dense_tc.cu

template <int EPI, bool F16, bool PREDICT>
static tsvm_status launch_pair_kernel(tsvm_km *km, const InstancePlanes &X, const RowPlanes &W, int m, float *out,
                                      long long ld_out, const PredictArgs &pa, const RowsExtra &ex, cudaStream_t st) {
    auto kernel = dense_rows_tc2_kernel<EPI, F16, PREDICT>;
    constexpr uint32_t smem_bytes = PREDICT ? tc2::SMEM_BYTES_PREDICT : tc2::SMEM_BYTES;
    static int clusters_of_device[MAX_DEVICES] = {0};      // per instantiation and per device ordinal
    int dev = 0;
    TSVM_CUDA(cudaGetDevice(&dev));
    int &max_clusters = clusters_of_device[dev & (MAX_DEVICES - 1)];
    if (!max_clusters) {
        int sms = 0;
        TSVM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        TSVM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes));
        cudaLaunchConfig_t probe = {};
        cudaLaunchAttribute pattr[1];
        pattr[0].id = cudaLaunchAttributeClusterDimension;
        pattr[0].val.clusterDim.x = 2; pattr[0].val.clusterDim.y = 1; pattr[0].val.clusterDim.z = 1;
        probe.gridDim = dim3(sms & ~1); probe.blockDim = dim3(tc2::THREADS); probe.dynamicSmemBytes = smem_bytes;
        probe.attrs = pattr; probe.numAttrs = 1;
        int nc = 0;
        if (cudaOccupancyMaxActiveClusters(&nc, kernel, &probe) != cudaSuccess || nc < 1) {
            cudaGetLastError();
            nc = sms / 2;
        }
        max_clusters = nc;
    }
    CUtensorMap mxh, mxl, mwh, mwl;
    const int len = km->plane_ld;
    TSVM_TRY(make_map(&mxh, X.hi, X.n, len, len, tc2::BM, F16));
    TSVM_TRY(make_map(&mxl, X.lo, X.n, len, len, tc2::BM, F16));
    TSVM_TRY(make_map(&mwh, W.hi, m, len, len, tc2::BN_HALF, F16));
    TSVM_TRY(make_map(&mwl, W.lo, m, len, len, tc2::BN_HALF, F16));
    const int n_items = ceil_div(X.n, 2 * tc2::BM) * ceil_div(m, tc2::BN);
    int avail = max_clusters - km->reserve_clusters;     // SM pairs left free for a concurrent stream
    if (avail < 1) avail = 1;
    const int clusters = n_items < avail ? n_items : avail;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * clusters); cfg.blockDim = dim3(tc2::THREADS); cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st; cfg.attrs = attr; cfg.numAttrs = 1;
    TSVM_CUDA(cudaLaunchKernelEx(&cfg, kernel, mxh, mxl, mwh, mwl, X.n, m, len, X.sd, W.sd, X.unscale, W.unscale,
                                 km->fn, out, ld_out, km->status_dev, pa, ex));
    count_launch();
    return TSVM_OK;
}

template <bool PREDICT>
static tsvm_status launch_pair_any(tsvm_km *km, const InstancePlanes &X, const RowPlanes &W, int m, float *out,
                                   long long ld_out, const PredictArgs &pa, const RowsExtra &ex, cudaStream_t st) {
    TSVM_REQUIRE(km->plane_kind == 1 || km->plane_kind == 2, "tensor engine: operand planes are not built");
    const int epi = epilogue_kind(km->fn);
    if (km->plane_kind == 2) {
        if (epi == EPI_RBF) return launch_pair_kernel<EPI_RBF, true, PREDICT>(km, X, W, m, out, ld_out, pa, ex, st);
        if (epi == EPI_LINEAR) return launch_pair_kernel<EPI_LINEAR, true, PREDICT>(km, X, W, m, out, ld_out, pa, ex, st);
        return launch_pair_kernel<EPI_GENERIC, true, PREDICT>(km, X, W, m, out, ld_out, pa, ex, st);
    }
    if (epi == EPI_RBF) return launch_pair_kernel<EPI_RBF, false, PREDICT>(km, X, W, m, out, ld_out, pa, ex, st);
    if (epi == EPI_LINEAR) return launch_pair_kernel<EPI_LINEAR, false, PREDICT>(km, X, W, m, out, ld_out, pa, ex, st);
    return launch_pair_kernel<EPI_GENERIC, false, PREDICT>(km, X, W, m, out, ld_out, pa, ex, st);
}

// Kernel values of the m staged requested rows against a set of instances given by its operand planes
// (kind 1 = TF32 words, 2 = row-scaled FP16, the handle's plane kind), self dots and 1/scale.
tsvm_status launch_dense_tc2_planes(tsvm_km *km, const InstancePlanes &X, const RowPlanes &W, int m, float *out,
                                    long long ld_out, cudaStream_t st) {
    return launch_pair_any<false>(km, X, W, m, out, ld_out, PredictArgs{}, RowsExtra{km->rows_m_dev, km->rows_slot_dev}, st);
}

// Prediction form: the m staged rows are test rows, the kernel matrix holds the support vectors; adds
// sum_sv coef * K(sv, test row) to dec_dev[r * n_pairs + pair] (preset by the caller) without writing K.
tsvm_status launch_dense_tc2_predict(tsvm_km *km, int m, const double *coef_dev, const int *sv_class_dev,
                                     int n_classes, double *dec_dev, cudaStream_t st) {
    const InstancePlanes all{km->Xhi, km->Xlo, km->self_dot, km->x_unscale, km->n};
    const RowPlanes staged{km->Whi, km->Wlo, km->sd_rows, km->w_unscale};
    const PredictArgs pa{coef_dev, sv_class_dev, dec_dev, n_classes, n_classes * (n_classes - 1) / 2};
    return launch_pair_any<true>(km, all, staged, m, nullptr, 0, pa, RowsExtra{nullptr, nullptr}, st);
}

// Requested rows = the m rows staged in the handle's scratch.
tsvm_status launch_dense_tc2_on(tsvm_km *km, const InstancePlanes &X, int m, float *out, long long ld_out,
                                cudaStream_t st) {
    const RowPlanes staged{km->Whi, km->Wlo, km->sd_rows, km->w_unscale};
    return launch_dense_tc2_planes(km, X, staged, m, out, ld_out, st);
}

// The same against all instances of the kernel matrix.
tsvm_status launch_dense_tc2(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st) {
    const InstancePlanes all{km->Xhi, km->Xlo, km->self_dot, km->x_unscale, km->n};
    return launch_dense_tc2_on(km, all, m, out, ld_out, st);
}

}  // namespace tsvm
