/*
 * thundersvm_b200 - C ABI of the B200 (sm_100a) implementation of ThunderSVM's training and
 * prediction hot path: KernelMatrix rows, the batched SMO solver and the prediction
 * contraction.
 *
 * Conventions
 *   - Every entry point returns a tsvm_status (0 = success). No C++ exception and no STL
 *     type crosses this boundary; tsvm_last_error() returns the message of the calling
 *     thread's last failure.
 *   - Pointers named *_dev are device pointers on the current CUDA device, *_host are host
 *     pointers. `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *   - Types follow the reference (include/thundersvm/thundersvm.h:16-22): feature and
 *     kernel values are float, alpha / f / rho / coefficients / decision values are double,
 *     labels and ids are int.
 *   - Kernel rows are written row-major, out[i * ld + j] = K(x_idx[i], x_j), the layout the
 *     reference's consumers read (src/thundersvm/kernel/smo_kernel.cu:62,298).
 *   - Handles own every device allocation they make; there is no process-global device
 *     state.
 */
#ifndef THUNDERSVM_B200_H
#define THUNDERSVM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int tsvm_status;
enum {
    TSVM_OK = 0,
    TSVM_ERR_INVALID = 1,     /* bad argument (the reference CHECK-fails / LOG(FATAL)s here)   */
    TSVM_ERR_CUDA = 2,        /* CUDA runtime / driver error                                    */
    TSVM_ERR_OOM = 3,         /* device allocation failed (reference: std::bad_alloc,           */
                              /* include/thundersvm/util/common.h:33-39)                        */
    TSVM_ERR_DEVICE = 4,      /* a kernel reported an error status (bounded wait ran out, ...)  */
    TSVM_ERR_UNSUPPORTED = 5
};

/* SvmParam::KERNEL_TYPE (include/thundersvm/svmparam.h:35-37) */
enum { TSVM_LINEAR = 0, TSVM_POLY = 1, TSVM_RBF = 2, TSVM_SIGMOID = 3, TSVM_PRECOMPUTED = 4 };
/* which solver: CSMOSolver, NuSMOSolver(for_svr=false), NuSMOSolver(for_svr=true) */
enum { TSVM_SOLVER_C = 0, TSVM_SOLVER_NU_SVC = 1, TSVM_SOLVER_NU_SVR = 2 };
/* where a caller's buffer lives */
enum { TSVM_HOST = 0, TSVM_DEVICE = 1 };

const char *tsvm_last_error(void);
/* ABI version, bumped on any signature change. */
int tsvm_abi_version(void);
/* Device and pinned-host memory released by destroyed handles is kept for the next handle of the same
 * size (the reference frees and reallocates per binary sub-problem); this returns it to the driver. */
void tsvm_release_cached_memory(void);

/* ------------------------------------------------------------------------------------------
 * KernelMatrix  (replaces include/thundersvm/kernelmatrix.h:46-72,
 *                src/thundersvm/kernelmatrix.cpp:183-316)
 * ---------------------------------------------------------------------------------------- */
typedef struct tsvm_km tsvm_km;

/* Constructor for dense instances: X is n x d row-major with row stride ld (floats).
 * loc = TSVM_HOST: X is copied to the device. loc = TSVM_DEVICE: if ld is a multiple of 4 and
 * X is 16-byte aligned the buffer is used in place (the caller keeps it alive), else copied.
 * Computes self dots (double accumulate, float store) and the diagonal as
 * kernelmatrix.cpp:194-247 does. Replaces KernelMatrix::KernelMatrix (kernelmatrix.cpp:183). */
tsvm_status tsvm_km_create_dense(const float *X, int n, int d, int ld, int loc, int kernel_type, int degree,
                                 float gamma, float coef0, void *stream, tsvm_km **out);

/* Constructor for CSR instances (0-based column ids < d, ascending inside a row).
 * Replaces KernelMatrix::KernelMatrix + CSR_DenseCSR (kernelmatrix.cpp:16-249). */
tsvm_status tsvm_km_create_csr(const float *val, const int *row_ptr, const int *col, int n, int d, int loc,
                               int kernel_type, int degree, float gamma, float coef0, void *stream,
                               tsvm_km **out);

void tsvm_km_destroy(tsvm_km *km);

int tsvm_km_n_instances(const tsvm_km *km);   /* KernelMatrix::n_instances, kernelmatrix.h:64 */
int tsvm_km_n_features(const tsvm_km *km);    /* KernelMatrix::n_features,  kernelmatrix.h:66 */
long long tsvm_km_nnz(const tsvm_km *km);     /* KernelMatrix::nnz,         kernelmatrix.h:68 */
int tsvm_km_is_dense(const tsvm_km *km);

/* Device pointers owned by the handle: diag()[n] (KernelMatrix::diag, kernelmatrix.cpp:314)
 * and the self dots [n]. */
const float *tsvm_km_diag_dev(const tsvm_km *km);
const float *tsvm_km_self_dot_dev(const tsvm_km *km);

/* q rows of the kernel matrix: out_dev[i * ld_out + j] = K(x_idx[i], x_j), j < n.
 * Replaces KernelMatrix::get_rows(idx, kernel_rows) (kernelmatrix.cpp:251-279) and the
 * svm_kernel:: calls under it (get_working_set_ins, dns_csr_mul, dns_dns_mul, RBF_kernel,
 * poly_kernel, sigmoid_kernel; include/thundersvm/kernel/kernelmatrix_kernel.h:13-66). */
tsvm_status tsvm_km_rows_by_index(tsvm_km *km, const int *idx_dev, int q, float *out_dev, long long ld_out,
                                  void *stream);

/* Kernel values of m new instances against the stored ones: out_dev[r * ld_out + j].
 * Features with id >= n_features are ignored in the product but counted in the test self
 * dot, as the reference does. Replaces KernelMatrix::get_rows(instances, kernel_rows)
 * (kernelmatrix.cpp:281-312, 385-406). The stored matrix and the batch may differ in
 * storage (dense / CSR). */
tsvm_status tsvm_km_rows_by_instances_dense(tsvm_km *km, const float *T_dev, int m, int dt, int ldt, float *out_dev,
                                            long long ld_out, void *stream);
tsvm_status tsvm_km_rows_by_instances_csr(tsvm_km *km, const float *tval_dev, const int *trow_ptr_dev,
                                          const int *tcol_dev, int m, long long tnnz, float *out_dev,
                                          long long ld_out, void *stream);

/* Kernel rows for m explicit feature rows T (m x n_features, row stride ldt) whose self dots the caller
 * supplies (sd_T_dev[m]); dense kernel matrices only. Used where the requested rows live on another
 * GPU: the column-sharded driver ships the working set's feature rows and self dots to every shard,
 * and each shard computes K(rows, its own instances) - the values are then identical to
 * tsvm_km_rows_by_index on one GPU. */
tsvm_status tsvm_km_rows_for_features_dense(tsvm_km *km, const float *T_dev, int ldt, const float *sd_T_dev, int m,
                                            float *out_dev, long long ld_out, void *stream);

/* Selects the dense kernel-row engine: 0 = automatic (default: engine 4, or FP32 CUDA-core tiles when
 * there are at most 32 features, where a k loop of one slab gives the tensor core nothing to
 * pipeline), 1 = FP32 CUDA-core tiles, 3 = tcgen05 CTA pairs on two TF32 planes (2 is accepted as an
 * alias), 4 = tcgen05 CTA pairs on two row-scaled FP16 planes (every row is multiplied by a power of
 * two that brings its largest magnitude to [2^14, 2^15) before the split; same accuracy class as
 * engine 3 at twice the tensor-core rate and half the operand bytes). The operand planes are built on
 * the first call that needs them; changing the engine rebuilds them. On a CSR matrix the setting is
 * ignored. */
tsvm_status tsvm_km_set_dense_engine(tsvm_km *km, int engine);

/* ------------------------------------------------------------------------------------------
 * Batched SMO solver (replaces include/thundersvm/solver/csmosolver.h:16-17,
 *                     include/thundersvm/solver/nusmosolver.h:15,
 *                     src/thundersvm/solver/csmosolver.cpp:10-239, nusmosolver.cpp:9-136)
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    long long outer_iters;      /* "global iter" of csmosolver.cpp:103-105                  */
    long long local_iters;      /* "total local iter"                                        */
    double final_diff;          /* last diff[0] (global maximal violation)                   */
    double objective;           /* calculate_obj, csmosolver.cpp:227-239 (before nu scaling) */
    double seconds_select;      /* host-observed phase times, seconds                        */
    double seconds_rows;
    double seconds_local;
    double seconds_update;
    double seconds_total;
    long long kernel_rows;      /* rows of length n delivered by get_rows (computed or cached) */
    long long gpu_launches;     /* kernels launched by this call                             */
    long long cache_hits;       /* delivered rows that were found in the kernel-row cache    */
    long long cache_misses;     /* delivered rows that the engine computed                   */
    long long cache_rows;       /* capacity of the cache, rows                               */
    long long row_blocks;       /* engine row blocks a cache-less solver would have computed */
    long long row_blocks_saved; /* ... of which the cache made this many unnecessary         */
} tsvm_solve_stats;

/* Kernel-row cache. The solver's row buffer holds as many kernel rows as this budget allows (at least the
 * working set plus one batch of new rows, at most one row per instance) and keeps the least recently
 * used ones across outer iterations; a requested row that is still there is not computed again. The
 * reference keeps only the previous iteration's rows (src/thundersvm/solver/csmosolver.cpp:33-42,69-76).
 * bytes < 0 restores the default (the environment variable TSVM_ROW_CACHE_MB if set, else 45 % of the
 * device's memory), 0 keeps no more than the minimum. Applies to solvers created afterwards. Results do
 * not depend on the budget: a cached row holds the values the engine would compute again. */
void tsvm_set_row_cache_bytes(long long bytes);

/* CSMOSolver::solve / NuSMOSolver::solve. y_dev[n] (+1/-1), alpha_dev[n] and f_dev[n] are
 * read and updated in place on the device; *rho_host receives rho. max_iter = -1 means no
 * limit on outer iterations (csmosolver.cpp:110). stats_host may be NULL. */
tsvm_status tsvm_smo_solve(tsvm_km *km, int solver_kind, const int *y_dev, double *alpha_dev, double *f_dev,
                           double eps, double Cp, double Cn, int ws_size, int max_iter, double *rho_host,
                           tsvm_solve_stats *stats_host, void *stream);

/* The same solver as an object, for callers that drive the outer loop themselves: create
 * (allocates the row buffer and runs init_f, csmosolver.cpp:189-214), iterate n outer iterations
 * (stops early and sets *done_host when the termination rules of csmosolver.cpp:86-111 fire),
 * finish (rho, objective, statistics; nu-SVC scaling), destroy. */
typedef struct tsvm_solver tsvm_solver;
tsvm_status tsvm_solver_create(tsvm_km *km, int solver_kind, const int *y_dev, double *alpha_dev, double *f_dev,
                               double eps, double Cp, double Cn, int ws_size, void *stream, tsvm_solver **out);
tsvm_status tsvm_solver_iterate(tsvm_solver *solver, int n_iters, int *done_host);
tsvm_status tsvm_solver_finish(tsvm_solver *solver, double *rho_host, tsvm_solve_stats *stats_host);
/* Counters and phase times so far (objective is not evaluated: NaN). */
tsvm_status tsvm_solver_get_stats(const tsvm_solver *solver, tsvm_solve_stats *stats_host);
/* Switches the overlapped outer iteration on (default) or off. Overlapped, the q full kernel rows are
 * computed on the caller's stream while the local solver runs on an internal second stream, fed by a
 * small extra launch that computes the q new rows of the ws x ws block first; it applies to dense data on
 * the CTA-pair tensor engine and gives bit-identical results (the block's values are computed by the same
 * arithmetic either way). No counterpart in the reference, whose steps run one after the other
 * (csmosolver.cpp:59-120). */
tsvm_status tsvm_solver_set_overlap(tsvm_solver *solver, int enable);
void tsvm_solver_destroy(tsvm_solver *solver);

/* ---- Column-sharded solver: the per-rank device work of CSMOSolver / NuSMOSolver::solve -----------
 * One large binary problem whose instances (columns of the kernel matrix) are split over `world`
 * processes, one GPU each: this rank owns instances [lo, lo + n_local) - km_local, y, alpha, f are
 * its slices. The reference has no multi-GPU form of this loop (csmosolver.cpp:59-120 runs on one
 * device); the steps and their results are the same, bit for bit, as tsvm_solver_* on one GPU.
 * One outer iteration is three calls with the caller's collectives in between (any library; the
 * buffers are plain device memory the caller allocated and passed to tsvm_shard_create):
 *   tsvm_shard_candidates  -> cand_f / cand_id hold lists x want entries (global ids);
 *                             all-gather them, rank-major, into all_f / all_id
 *   tsvm_shard_select      -> the same merge on every rank; rows_contrib ([n_new][dp + 4] floats,
 *                             dp = round_up(n_features, 4): feature row, self dot, diagonal) and
 *                             state_contrib ([ws][3] doubles: y, f, alpha) hold this rank's share,
 *                             zeros for members it does not own; all-reduce (sum) both
 *   tsvm_shard_iterate     -> kernel rows of the new members against the own columns, the ws x ws
 *                             block and the local solver (replicated, deterministic), f / alpha
 *                             update of the own slice, the reference's stopping rules
 * Buffer sizes: cand_* lists_max(4) * ws entries, all_* world * 4 * ws, rows_contrib ws * (dp + 4),
 * state_contrib ws * 3. Needs dense data with more than 32 features (CTA-pair tensor engine). */
typedef struct tsvm_shard tsvm_shard;
tsvm_status tsvm_shard_create(tsvm_km *km_local, int solver_kind, const int *y_dev, double *alpha_dev, double *f_dev,
                              int n_total, int lo, double eps, double Cp, double Cn, int ws_size, int world,
                              double *cand_f_dev, int *cand_id_dev, double *all_f_dev, int *all_id_dev,
                              float *rows_contrib_dev, double *state_contrib_dev, void *stream, tsvm_shard **out);
tsvm_status tsvm_shard_candidates(tsvm_shard *shard, int *lists_host, int *want_host);
tsvm_status tsvm_shard_select(tsvm_shard *shard, int *n_new_host);
tsvm_status tsvm_shard_iterate(tsvm_shard *shard, int *done_host);
/* The same iteration with the exchange steps run by the library itself: NCCL is looked up at run time in
 * the process (libnccl.so.2; the library does not link it). Rank 0 asks for a 128-byte unique id
 * (ncclGetUniqueId), the caller distributes it by any means, every rank creates a communicator
 * (ncclCommInitRank, a collective call; the handle may serve any number of shard solvers of the same ranks,
 * one at a time), attaches it, and tsvm_shard_step then runs candidates -> all-gather -> select ->
 * all-reduce -> iterate on the solver's stream without host work in between. */
int tsvm_nccl_unique_id(void *id128_host);
tsvm_status tsvm_nccl_comm_create(const void *id128_host, int rank, int world, void **comm_out);
void tsvm_nccl_comm_destroy(void *comm);
tsvm_status tsvm_shard_attach_nccl(tsvm_shard *shard, void *comm);
tsvm_status tsvm_shard_step(tsvm_shard *shard, int *done_host);
/* Up to n_iters such iterations. The termination rules run on the device, as in tsvm_solver_iterate: several
 * iterations (eight, TSVM_SYNC_EVERY) are queued between reads of the verdict, collectives included - every rank
 * must call it with the same n_iters. Stops early when the solve is done. */
tsvm_status tsvm_shard_run(tsvm_shard *shard, int n_iters, int *done_host);
tsvm_status tsvm_shard_get_stats(const tsvm_shard *shard, tsvm_solve_stats *stats_host);
void tsvm_shard_destroy(tsvm_shard *shard);

/* The 13 partial reductions rho and the objective are made of (csmosolver.cpp:167-187,227-239;
 * nusmosolver.cpp:9-46), over the n instances given: out13_dev[0..12] = n_free(y>0), sum f over them,
 * n_free(y<0), sum f over them, sum_i alpha_i - (f_i + y_i) alpha_i y_i / 2, then min f over I_up and
 * max f over I_low for y>0 and for y<0, then max f over I_up and min f over I_low for y>0 and y<0.
 * Shards combine them (sums, mins, maxes) into the global rho and objective. */
tsvm_status tsvm_rho_partials(int n, const double *f_dev, const double *alpha_dev, const int *y_dev, double Cp,
                              double Cn, double *out13_dev, void *stream);

/* SvmModel::get_working_set_size (src/thundersvm/model/svmmodel.cpp:437-451) with the
 * memory budget in bytes. Returns the working-set size, or -1 when the budget is already
 * exceeded (the reference throws std::bad_alloc there). */
int tsvm_working_set_size(int n_instances, int n_features, size_t max_mem_bytes, size_t used_bytes);

/* ---- the solver's steps, one entry point each (used by the column-sharded multi-GPU
 *      driver and by the unit tests) ---------------------------------------------------- */
typedef struct tsvm_ws tsvm_ws;   /* scratch for working-set selection */
tsvm_status tsvm_ws_create(int n_max, int ws_max, tsvm_ws **out);
void tsvm_ws_destroy(tsvm_ws *w);

/* Candidate lists for the working set: for each of the solver's pointer walks
 * (C: I_up ascending f, I_low descending f; nu: the same per class) the first `want`
 * instances in (f, id) order that are not flagged in in_ws_dev[n] (0/1 bytes, may be NULL).
 * cand_f_dev[list * want + r], cand_id_dev[...] (id -1 = list exhausted). id_offset is
 * added to every reported id (a shard's first global column). Replaces svm_kernel::sort_f
 * (smo_kernel.cu:312-315). */
tsvm_status tsvm_ws_candidates(tsvm_ws *w, int solver_kind, int n, const double *f_dev, const double *alpha_dev,
                               const int *y_dev, const unsigned char *in_ws_dev, double Cp, double Cn, int want,
                               int id_offset, double *cand_f_dev, int *cand_id_dev, void *stream);

/* Alternating merge of the candidate lists (each of length `len`, sorted as above) into
 * `want` distinct ids: CSMOSolver::select_working_set (csmosolver.cpp:123-165) /
 * NuSMOSolver::select_working_set (nusmosolver.cpp:48-118) restricted to the candidates. */
tsvm_status tsvm_ws_merge(tsvm_ws *w, int solver_kind, const double *cand_f_dev, const int *cand_id_dev, int len,
                          int want, int *out_ids_dev, void *stream);
/* The same in two steps that scale with the number of ranks: every rank sorts its own lists in place
 * (padding last), and the concatenation of the ranks' runs - len entries per list, in runs of seg_len -
 * is merged by rank computation (binary searches) instead of one sort of all candidates. */
tsvm_status tsvm_ws_sort_candidates(tsvm_ws *ws, int solver_kind, double *cand_f_dev, int *cand_id_dev, int len,
                                    void *stream);
tsvm_status tsvm_ws_merge_sorted(tsvm_ws *ws, int solver_kind, const double *cand_f_dev, const int *cand_id_dev,
                                 int len, int seg_len, int want, int *out_ids_dev, void *stream);

/* Full selection = candidates + merge on one device. */
tsvm_status tsvm_select_working_set(tsvm_ws *w, int solver_kind, int n, const double *f_dev,
                                    const double *alpha_dev, const int *y_dev, const unsigned char *in_ws_dev,
                                    double Cp, double Cn, int want, int *out_ids_dev, void *stream);

/* Allocation-free working-set selection. Same result as tsvm_select_working_set, but needs no tsvm_ws
 * and calls neither cudaMalloc / cudaFree nor any other allocating routine: its scratch (selection
 * state, radix histograms, candidate lists; 115,200 bytes) is a fixed array inside the library image,
 * resident on every GPU that loads the library. It has no counterpart in the reference. It is meant
 * for callers that must not allocate at the point where they pick a working set: a solver loop that
 * has handed all device memory to its own pool (a later cudaMalloc would fail or fragment it), or a
 * latency-sensitive loop sharing the GPU with other streams, which a cudaMalloc would stall because
 * allocation synchronises the whole device.
 * Limits and rules: want <= TSVM_STATIC_WS_MAX (TSVM_ERR_INVALID with a message otherwise; n is
 * unlimited). The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and sets the shared-memory limits of the selection
 * kernels (cudaFuncSetAttribute) - make that first call outside any stream capture. All calls on a
 * device share the one array: it still holds the previous call's contents when a call starts (the
 * entry point clears what must start at zero itself), and two calls that overlap on the GPU - from
 * different streams or threads - race on it; serialise them. */
#define TSVM_STATIC_WS_MAX 1024
tsvm_status tsvm_select_working_set_static(int solver_kind, int n, const double *f_dev, const double *alpha_dev,
                                           const int *y_dev, const unsigned char *in_ws_dev, double Cp,
                                           double Cn, int want, int *out_ids_dev, void *stream);

/* Local SMO on one working set: svm_kernel::c_smo_solve / nu_smo_solve
 * (smo_kernel.cu:28-287). kww_dev is the ws x ws block K(x_ws[a], x_ws[b]) (row-major,
 * stride ws); y/f/alpha/diag_ws_dev hold the working set's values in slot order. Outputs:
 * alpha_ws_dev (updated), alpha_diff_dev[ws] = -(a - a_old) * y, diff_dev[0] = first gap,
 * diff_dev[1] = #local iterations. */
tsvm_status tsvm_local_smo(int solver_kind, int ws_size, const float *kww_dev, const float *diag_ws_dev,
                           const int *y_ws_dev, const double *f_ws_dev, double *alpha_ws_dev,
                           double *alpha_diff_dev, double Cp, double Cn, double eps, int max_iter, double *diff_dev,
                           void *stream);

/* f[j] -= sum_i alpha_diff[i] * rows[i * ld + j] (zero alpha_diff rows skipped, double
 * accumulation): svm_kernel::update_f (smo_kernel.cu:289-310). */
tsvm_status tsvm_update_f(double *f_dev, int n, const double *alpha_diff_dev, int ws_size, const float *rows_dev,
                          long long ld, void *stream);

/* ------------------------------------------------------------------------------------------
 * Prediction (replaces SvmModel::predict_dec_values, src/thundersvm/model/svmmodel.cpp:74-117
 *             and svm_kernel::sum_kernel_values, kernelmatrix_kernel.cu:69-97,154-162)
 * ---------------------------------------------------------------------------------------- */

/* dec_dev[r * nb + k] = sum over the support vectors of pair k of coef * K(sv, x_r) - rho[k],
 * nb = n_classes (n_classes - 1) / 2, pairs ordered (0,1),(0,2),...; coef_dev is the
 * (n_classes - 1) x n_sv layout of include/thundersvm/model/svmmodel.h:155-164, sv_count_host
 * the per-class support-vector counts, rho_dev[nb]. km_sv holds the support vectors. The test
 * batch is dense (T_dev != NULL) or CSR. Batching over the test rows is internal. With dense support
 * vectors of more than 32 features the coefficient sums are part of the contraction's epilogue (FP32
 * partial sums over 128 support vectors, combined in FP64) and the test x SV kernel block is never stored;
 * otherwise it is computed in slabs of at most max_mem_bytes (0 = a quarter of the free memory). */
tsvm_status tsvm_predict_dec(tsvm_km *km_sv, const double *coef_dev, const int *sv_count_host,
                             const double *rho_dev, int n_classes, int m, const float *T_dev, int dt, int ldt,
                             const float *tval_dev, const int *trow_ptr_dev, const int *tcol_dev, long long tnnz,
                             double *dec_dev, size_t max_mem_bytes, void *stream);

/* The same contraction with the vote on the device: labels_dev[r] = index of the winning class (first
 * maximum wins), and no decision value leaves the device - they live in a scratch of one slab of test rows.
 * Replaces SvmModel::predict_dec_values_instant (src/thundersvm/model/svmmodel.cpp:119-154) and
 * svm_kernel::sum_kernel_values_instant (kernelmatrix_kernel.cu:99-138,164-172), which the reference uses
 * for models with more than 10,000 class pairs (svc.cpp:180-181). */
tsvm_status tsvm_predict_labels(tsvm_km *km_sv, const double *coef_dev, const int *sv_count_host,
                                const double *rho_dev, int n_classes, int m, const float *T_dev, int dt, int ldt,
                                const float *tval_dev, const int *trow_ptr_dev, const int *tcol_dev, long long tnnz,
                                int *labels_dev, size_t max_mem_bytes, void *stream);

/* SVC::predict_label voting (src/thundersvm/model/svc.cpp:265-289): out_dev[r] = index of the
 * winning class. */
tsvm_status tsvm_vote(const double *dec_dev, int m, int n_classes, int *out_dev, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* THUNDERSVM_B200_H */
