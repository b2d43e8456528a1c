// Batched SMO solver on the device: working-set selection (radix top-k over (f, id) keys),
// the one-CTA local solver, the fused f update and the outer loop with the reference's
// termination rules. Reference behaviour: src/thundersvm/solver/csmosolver.cpp:10-239,
// src/thundersvm/solver/nusmosolver.cpp:9-136, src/thundersvm/kernel/smo_kernel.cu:28-315.
#include "common.cuh"
#include <cooperative_groups.h>
#include <chrono>
#include <limits.h>
#include <string.h>
#include <stdlib.h>
#include <dlfcn.h>
#include <vector>

namespace tsvm {

// =================================================================================================
// Working-set selection
// =================================================================================================
// The reference sorts all n f-values every outer iteration (smo_kernel.cu:312-315) and then walks
// the sorted ids from both ends on the host (csmosolver.cpp:123-165). Only the first `want`
// eligible instances of every walk can ever be taken, so the device keeps, per walk ("list"),
// the `want` smallest 96-bit keys (f-order, id) among the eligible instances:
//   C-SMO : list 0 = I_up ascending (f, id);      list 1 = I_low descending (f, id)
//   nu-SMO: lists 0/1 = I_up for y>0 / y<0;       lists 2/3 = I_low for y>0 / y<0
// found with a 12-bit radix select of up to 8 passes, followed by a compaction (select_fused_kernel below).
// One pass = histogram of the current digit over the eligible instances that match the prefix, all lists in
// one sweep over the data; the last block to finish picks, per list, the digit that holds the wanted rank. A
// list whose threshold digit holds few enough instances for the whole digit to fit the candidate capacity
// `cap` is resolved on the spot (the threshold becomes "everything up to and including this digit" and the
// exact order is left to the sort of the candidates), so that in practice two passes do the work.

constexpr int RADIX_BITS = 12, RADIX_BINS = 1 << RADIX_BITS, RADIX_PASSES = 8, MAX_LISTS = 4;
typedef unsigned __int128 key96_t;

struct SelectState {            // one per list, lives in device memory
    unsigned long long prefix_hi;   // bits 95..32 of the threshold key found so far
    unsigned int prefix_lo;         // bits 31..0
    int k_rem;                      // rank still to resolve inside the current prefix
    int take_all;                   // fewer candidates than wanted: take every one
    int count;                      // compaction cursor
    int resolved;                   // the threshold is final: later radix passes skip this list
};

__device__ __forceinline__ int list_count(int solver_kind) { return solver_kind == TSVM_SOLVER_C ? 2 : 4; }

// Is instance (a, y) eligible for list l?
__device__ __forceinline__ bool in_list(int solver_kind, int l, double a, int y, double Cp, double Cn) {
    if (solver_kind == TSVM_SOLVER_C) return l == 0 ? in_I_up(a, y, Cp, Cn) : in_I_low(a, y, Cp, Cn);
    const bool pos = (l & 1) == 0;
    if (pos != (y > 0)) return false;
    return l < 2 ? in_I_up(a, y, Cp, Cn) : in_I_low(a, y, Cp, Cn);
}
__device__ __forceinline__ bool list_ascending(int solver_kind, int l) {
    return solver_kind == TSVM_SOLVER_C ? l == 0 : l < 2;
}
__device__ __forceinline__ key96_t make_key(bool asc, double f, unsigned id) {
    unsigned long long h = ordered_key(f);
    if (!asc) { h = ~h; id = ~id; }
    return ((key96_t) h << 32) | id;
}

// ---- merge: sort every candidate list, keep its first `want`, then the reference's alternating
// walk with "already taken" checks (csmosolver.cpp:123-165 / nusmosolver.cpp:48-118). ------------
constexpr int MERGE_THREADS = 1024, MERGE_MAX_LEN = 8192, MERGE_MAX_WANT = 1024, HASH_SLOTS = 4096;
constexpr int MERGE_JOINT_MAX = 2048;          // longest lists that merge_lists sorts side by side

__device__ __forceinline__ bool key_less(unsigned long long ah, unsigned al, unsigned long long bh, unsigned bl) {
    return ah < bh || (ah == bh && al < bl);
}

__device__ void merge_lists(int solver_kind, const double *__restrict__ cand_f, const int *__restrict__ cand_id, int len,
                            int want, int *__restrict__ out_ids, int *__restrict__ out_count, int seg_len,
                            unsigned char *smem) {
    const int lists = list_count(solver_kind);
    int P = 1;
    while (P < len) P <<= 1;
    // layout: sort keys (P x 12 B), then per list: top ids / partner positions / taken flags
    unsigned long long *kh = reinterpret_cast<unsigned long long *>(smem);
    unsigned int *kl = reinterpret_cast<unsigned int *>(kh + P);
    int *top_id = reinterpret_cast<int *>(kl + P);                 // [lists][want]
    short *partner = reinterpret_cast<short *>(top_id + MAX_LISTS * MERGE_MAX_WANT);   // [lists][want]
    unsigned char *taken = reinterpret_cast<unsigned char *>(partner + MAX_LISTS * MERGE_MAX_WANT);
    int *hash_id = reinterpret_cast<int *>(taken + MAX_LISTS * MERGE_MAX_WANT);        // [HASH_SLOTS]
    short *hash_pos = reinterpret_cast<short *>(hash_id + HASH_SLOTS);
    __shared__ int top_len[MAX_LISTS];
    __shared__ unsigned long long last_fkey[MAX_LISTS];
    __shared__ int real_total;
    const int tid = threadIdx.x;

    // Lists that are not made of sorted runs and fit the shared memory side by side are sorted together: every
    // step of the bitonic network handles all lists before its barrier (half the barriers for two lists).
    const bool joint = seg_len == 0 && P <= MERGE_JOINT_MAX;
    if (joint) {
        for (int l = 0; l < lists; ++l) {
            const bool asc = list_ascending(solver_kind, l);
            for (int e = tid; e < P; e += MERGE_THREADS) {
                unsigned long long h = ~0ull;
                unsigned lo = ~0u;
                if (e < len) {
                    const int id = __ldcg(cand_id + (size_t) l * len + e);
                    if (id >= 0) {
                        h = ordered_key(__ldcg(cand_f + (size_t) l * len + e));
                        lo = (unsigned) id;
                        if (!asc) { h = ~h; lo = ~lo; }
                    }
                }
                kh[(size_t) l * P + e] = h;
            }
        }
        // (kl follows all lists' kh)
        unsigned int *klj = reinterpret_cast<unsigned int *>(kh + (size_t) lists * P);
        for (int l = 0; l < lists; ++l) {
            const bool asc = list_ascending(solver_kind, l);
            for (int e = tid; e < P; e += MERGE_THREADS) {
                unsigned lo = ~0u;
                if (e < len) {
                    const int id = __ldcg(cand_id + (size_t) l * len + e);
                    if (id >= 0) lo = asc ? (unsigned) id : ~(unsigned) id;
                }
                klj[(size_t) l * P + e] = lo;
            }
        }
        __syncthreads();
        for (int k = 2; k <= P; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int w = tid; w < lists * (P >> 1); w += MERGE_THREADS) {
                    // comparison w of this step: list l, lower element e (bit j clear), partner e | j
                    const int l = w / (P >> 1), c = w - l * (P >> 1);
                    const int e = ((c & ~(j - 1)) << 1) | (c & (j - 1));
                    const int x = e | j;
                    unsigned long long *khl = kh + (size_t) l * P;
                    unsigned int *kll = klj + (size_t) l * P;
                    const bool up = (e & k) == 0;
                    if (key_less(khl[x], kll[x], khl[e], kll[e]) == up) {
                        unsigned long long th = khl[e]; khl[e] = khl[x]; khl[x] = th;
                        unsigned tl = kll[e]; kll[e] = kll[x]; kll[x] = tl;
                    }
                }
                __syncthreads();
            }
        int *top_id_j = reinterpret_cast<int *>(klj + (size_t) lists * P);
        top_id = top_id_j;
        partner = reinterpret_cast<short *>(top_id + MAX_LISTS * MERGE_MAX_WANT);
        taken = reinterpret_cast<unsigned char *>(partner + MAX_LISTS * MERGE_MAX_WANT);
        hash_id = reinterpret_cast<int *>(taken + MAX_LISTS * MERGE_MAX_WANT);
        hash_pos = reinterpret_cast<short *>(hash_id + HASH_SLOTS);
        for (int l = 0; l < lists; ++l) {
            const bool asc = list_ascending(solver_kind, l);
            const unsigned long long *khl = kh + (size_t) l * P;
            const unsigned int *kll = klj + (size_t) l * P;
            for (int e = tid; e < want; e += MERGE_THREADS) {
                int id = -1;
                if (e < P && !(khl[e] == ~0ull && kll[e] == ~0u)) id = (int) (asc ? kll[e] : ~kll[e]);
                top_id[l * MERGE_MAX_WANT + e] = id;
                partner[l * MERGE_MAX_WANT + e] = -1;
                taken[l * MERGE_MAX_WANT + e] = 0;
            }
        }
        __syncthreads();
        if (tid < lists) {
            const int l = tid;
            const bool asc = list_ascending(solver_kind, l);
            const unsigned long long *khl = kh + (size_t) l * P;
            int c = want < P ? want : P;
            int lo = 0, hi = c;
            while (lo < hi) { int mid = (lo + hi) >> 1; if (top_id[l * MERGE_MAX_WANT + mid] >= 0) lo = mid + 1; else hi = mid; }
            top_len[l] = lo;
            last_fkey[l] = lo > 0 ? (asc ? khl[lo - 1] : ~khl[lo - 1]) : 0ull;
        }
        __syncthreads();
    }

    for (int l = 0; l < lists && !joint; ++l) {
        const bool asc = list_ascending(solver_kind, l);
        for (int e = tid; e < P; e += MERGE_THREADS) {
            unsigned long long h = ~0ull;
            unsigned lo = ~0u;
            if (e < len) {
                const int id = __ldcg(cand_id + (size_t) l * len + e);      // written by other blocks: from L2
                if (id >= 0) {
                    h = ordered_key(__ldcg(cand_f + (size_t) l * len + e));
                    lo = (unsigned) id;
                    if (!asc) { h = ~h; lo = ~lo; }
                    // keep real keys distinct from the padding key
                }
            }
            kh[e] = h; kl[e] = lo;
        }
        __syncthreads();
        if (seg_len > 0) {
            // The list is a sequence of sorted runs (one per rank, padding last): an entry's place in the merged
            // order is its place in its own run plus, for every other run, the number of smaller keys there
            // (binary search; keys are distinct because ids are). No sort, a few microseconds for 8 x 512.
            const int nseg = len / seg_len;
            for (int e = tid; e < want; e += MERGE_THREADS) {
                top_id[l * MERGE_MAX_WANT + e] = -1;
                partner[l * MERGE_MAX_WANT + e] = -1;
                taken[l * MERGE_MAX_WANT + e] = 0;
            }
            if (tid == 0) real_total = 0;
            __syncthreads();
            if (tid < nseg) {                       // real entries of run tid: first padding key
                int lo_i = 0, hi_i = seg_len;
                while (lo_i < hi_i) {
                    const int mid = (lo_i + hi_i) >> 1;
                    const int e = tid * seg_len + mid;
                    if (kh[e] == ~0ull && kl[e] == ~0u) hi_i = mid; else lo_i = mid + 1;
                }
                atomicAdd(&real_total, lo_i);
            }
            __syncthreads();
            const int keep = real_total < want ? real_total : want;
            for (int e = tid; e < len; e += MERGE_THREADS) {
                const unsigned long long h = kh[e];
                const unsigned lo = kl[e];
                if (h == ~0ull && lo == ~0u) continue;
                const int r = e / seg_len;
                int rank = e - r * seg_len;
                for (int r2 = 0; r2 < nseg && rank < want; ++r2) {
                    if (r2 == r) continue;
                    int lo_i = 0, hi_i = seg_len;            // number of keys in run r2 below (h, lo)
                    while (lo_i < hi_i) {
                        const int mid = (lo_i + hi_i) >> 1;
                        const int x = r2 * seg_len + mid;
                        if (key_less(kh[x], kl[x], h, lo)) lo_i = mid + 1; else hi_i = mid;
                    }
                    rank += lo_i;
                }
                if (rank < want) {
                    top_id[l * MERGE_MAX_WANT + rank] = (int) (asc ? lo : ~lo);
                    if (rank == keep - 1) last_fkey[l] = asc ? h : ~h;
                }
            }
            if (tid == 0) { top_len[l] = keep; if (keep == 0) last_fkey[l] = 0ull; }
            __syncthreads();
            continue;
        }
        for (int k = 2; k <= P; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int e = tid; e < P; e += MERGE_THREADS) {
                    const int x = e ^ j;
                    if (x > e) {
                        const bool up = (e & k) == 0;
                        const bool lt = key_less(kh[x], kl[x], kh[e], kl[e]);
                        if (lt == up) {
                            unsigned long long th = kh[e]; kh[e] = kh[x]; kh[x] = th;
                            unsigned tl = kl[e]; kl[e] = kl[x]; kl[x] = tl;
                        }
                    }
                }
                __syncthreads();
            }
        for (int e = tid; e < want; e += MERGE_THREADS) {
            int id = -1;
            if (e < P && !(kh[e] == ~0ull && kl[e] == ~0u)) id = (int) (asc ? kl[e] : ~kl[e]);
            top_id[l * MERGE_MAX_WANT + e] = id;
            partner[l * MERGE_MAX_WANT + e] = -1;
            taken[l * MERGE_MAX_WANT + e] = 0;
        }
        __syncthreads();
        if (tid == 0) {
            int c = want < P ? want : P;
            // entries are sorted, padding last: count the real ones
            int lo = 0, hi = c;
            while (lo < hi) { int mid = (lo + hi) >> 1; if (top_id[l * MERGE_MAX_WANT + mid] >= 0) lo = mid + 1; else hi = mid; }
            top_len[l] = lo;
            // f-order key of the last kept entry: the list's largest f (ascending) / smallest f (descending)
            last_fkey[l] = lo > 0 ? (asc ? kh[lo - 1] : ~kh[lo - 1]) : 0ull;
        }
        __syncthreads();
    }

    // An instance sits in an "up" list and in the paired "low" list only if the up list's largest f is not
    // below the low list's smallest f. For large problems that never happens: no instance is then met twice,
    // the reference's alternating walk takes entry p of every list in round p, and the output position of
    // every entry follows from the list lengths alone.
    const int half = lists / 2;
    bool disjoint = true;
    for (int u = 0; u < half; ++u)
        if (top_len[u] > 0 && top_len[u + half] > 0 && !(last_fkey[u] < last_fkey[u + half])) disjoint = false;
    if (disjoint) {
        int total = 0;
        for (int l = 0; l < lists; ++l) total += top_len[l];
        const int got = total < want ? total : want;
        for (int e = tid; e < lists * want; e += MERGE_THREADS) {
            const int l = e / want, p = e - l * want;
            if (p >= top_len[l]) continue;
            int pos = 0;
            for (int o = 0; o < lists; ++o) pos += (top_len[o] < p ? top_len[o] : p) + ((o < l && top_len[o] > p) ? 1 : 0);
            if (pos < want) out_ids[pos] = top_id[l * MERGE_MAX_WANT + p];
        }
        for (int r = got + tid; r < want; r += MERGE_THREADS) out_ids[r] = -1;
        if (tid == 0 && out_count) *out_count = got;
        return;
    }

    // partner positions: an instance can sit in an "up" list and in the "low" list of the same
    // class. up list u pairs with low list u + lists/2.
    for (int u = 0; u < half; ++u) {
        const int lw = u + half;
        for (int s = tid; s < HASH_SLOTS; s += MERGE_THREADS) hash_id[s] = -1;
        __syncthreads();
        for (int e = tid; e < top_len[lw]; e += MERGE_THREADS) {
            const int id = top_id[lw * MERGE_MAX_WANT + e];
            unsigned s = ((unsigned) id * 2654435761u) >> 20;
            for (;;) {
                const int old = atomicCAS(&hash_id[s], -1, id);
                if (old == -1) { hash_pos[s] = (short) e; break; }
                s = (s + 1) & (HASH_SLOTS - 1);
            }
        }
        __syncthreads();
        for (int e = tid; e < top_len[u]; e += MERGE_THREADS) {
            const int id = top_id[u * MERGE_MAX_WANT + e];
            unsigned s = ((unsigned) id * 2654435761u) >> 20;
            for (;;) {
                const int cur = hash_id[s];
                if (cur == -1) break;
                if (cur == id) {
                    const short p = hash_pos[s];
                    partner[u * MERGE_MAX_WANT + e] = p;
                    partner[lw * MERGE_MAX_WANT + p] = (short) e;
                    break;
                }
                s = (s + 1) & (HASH_SLOTS - 1);
            }
        }
        __syncthreads();
    }

    if (tid == 0) {
        int ptr[MAX_LISTS] = {0, 0, 0, 0};
        int got = 0;
        bool progressed = true;
        while (got < want && progressed) {
            progressed = false;
            for (int l = 0; l < lists && got < want; ++l) {
                const int other = l < half ? l + half : l - half;
                int p = ptr[l];
                const int L = top_len[l];
                while (p < L) {
                    const short pp = partner[l * MERGE_MAX_WANT + p];
                    if (pp < 0 || !taken[other * MERGE_MAX_WANT + pp]) break;
                    ++p;
                }
                if (p < L) {
                    out_ids[got++] = top_id[l * MERGE_MAX_WANT + p];
                    taken[l * MERGE_MAX_WANT + p] = 1;
                    ++p;
                    progressed = true;
                }
                ptr[l] = p;
            }
        }
        if (out_count) *out_count = got;
        for (int r = got; r < want; ++r) out_ids[r] = -1;
    }
}

__global__ void __launch_bounds__(MERGE_THREADS)
select_merge_kernel(int solver_kind, const double *__restrict__ cand_f, const int *__restrict__ cand_id, int len,
                    int want, int *__restrict__ out_ids, int *__restrict__ out_count, int seg_len) {
    extern __shared__ unsigned char smem[];
    merge_lists(solver_kind, cand_f, cand_id, len, want, out_ids, out_count, seg_len, smem);
}

// Sorts a candidate list by its list key (padding, id -1, last): one block per list, bitonic in shared
// memory. The runs of several ranks can then be merged by rank computation instead of a sort.
__device__ void sort_list(int solver_kind, int l, const double *cand_f, const int *cand_id, int len, double *out_f,
                          int *out_id, int out_len, unsigned char *smem) {
    const int tid = threadIdx.x;
    int P = 1;
    while (P < len) P <<= 1;
    unsigned long long *kh = reinterpret_cast<unsigned long long *>(smem);
    unsigned int *kl = reinterpret_cast<unsigned int *>(kh + P);
    double *fv = reinterpret_cast<double *>(kl + P + (P & 1));          // the f values travel with their keys
    const bool asc = list_ascending(solver_kind, l);
    for (int e = tid; e < P; e += MERGE_THREADS) {
        unsigned long long h = ~0ull;
        unsigned lo = ~0u;
        double v = 0.0;
        if (e < len) {
            const int id = __ldcg(cand_id + (size_t) l * len + e);
            if (id >= 0) {
                v = __ldcg(cand_f + (size_t) l * len + e);
                h = ordered_key(v);
                lo = (unsigned) id;
                if (!asc) { h = ~h; lo = ~lo; }
            }
        }
        kh[e] = h; kl[e] = lo; fv[e] = v;
    }
    __syncthreads();
    for (int k = 2; k <= P; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int e = tid; e < P; e += MERGE_THREADS) {
                const int x = e ^ j;
                if (x > e) {
                    const bool up = (e & k) == 0;
                    if (key_less(kh[x], kl[x], kh[e], kl[e]) == up) {
                        unsigned long long th = kh[e]; kh[e] = kh[x]; kh[x] = th;
                        unsigned tl = kl[e]; kl[e] = kl[x]; kl[x] = tl;
                        double tv = fv[e]; fv[e] = fv[x]; fv[x] = tv;
                    }
                }
            }
            __syncthreads();
        }
    // the first out_len entries of the sorted list (out_len <= len; the output may be the input)
    for (int e = tid; e < out_len; e += MERGE_THREADS) {
        const bool pad = kh[e] == ~0ull && kl[e] == ~0u;
        out_f[(size_t) l * out_len + e] = pad ? 0.0 : fv[e];
        out_id[(size_t) l * out_len + e] = pad ? -1 : (int) (asc ? kl[e] : ~kl[e]);
    }
}

__global__ void __launch_bounds__(MERGE_THREADS)
select_sort_candidates_kernel(int solver_kind, const double *cand_f, const int *cand_id, int len, double *out_f,
                              int *out_id, int out_len) {
    extern __shared__ unsigned char smem[];
    sort_list(solver_kind, blockIdx.x, cand_f, cand_id, len, out_f, out_id, out_len, smem);
}

// ---- the whole selection as ONE cooperative launch -------------------------------------------------------
// init -> radix passes (as many as the data needs, decided on the device) -> compaction -> sort / merge of the
// candidates, with grid-wide barriers between the phases instead of one launch per phase. The launch is
// cooperative (all blocks resident), so the barriers cannot deadlock. Every block takes the same path
// through the barriers: the decisions between them depend only on state written before the previous barrier.
namespace cg = cooperative_groups;
constexpr int FUSED_THREADS = 1024;
enum { FUSED_CANDIDATES = 0, FUSED_MERGE = 1, FUSED_SORT = 2 };

struct SelectArgs {
    int solver_kind, n;
    const double *f, *alpha;
    const int *y;
    const unsigned char *in_ws;
    double Cp, Cn;
    SelectState *st;
    int *hist, *ticket;
    int want, cap, id_offset;
    double *cand_f;             // [lists][cap]
    int *cand_id;
    int mode;                   // FUSED_*
    int *out_ids, *out_count;   // FUSED_MERGE: the selected ids
    double *sorted_f;           // FUSED_SORT: the `want` best of every list, sorted, [lists][want]
    int *sorted_id;
    // optional rotation of the working set before the selection (plain solver): ids[0..q) <- ids[q..2q),
    // in-working-set flags of the leaving / staying members
    int *shift_ids;
    int shift_q;
    unsigned char *shift_flags;
    // optional: when *stop is non-zero the whole launch is a no-op (iterations queued past the end of a solve)
    const int *stop;
};

__device__ void merge_lists(int solver_kind, const double *cand_f, const int *cand_id, int len, int want, int *out_ids,
                            int *out_count, int seg_len, unsigned char *smem);
__device__ void sort_list(int solver_kind, int l, const double *cand_f, const int *cand_id, int len, double *out_f,
                          int *out_id, int out_len, unsigned char *smem);

__global__ void __launch_bounds__(FUSED_THREADS, 1) select_fused_kernel(const SelectArgs a) {
    extern __shared__ unsigned char fused_smem[];
    int *sh = reinterpret_cast<int *>(fused_smem);
    __shared__ int scan[256];
    __shared__ bool is_last;
    cg::grid_group grid = cg::this_grid();
    const int lists = list_count(a.solver_kind);
    // the selection state is written by other blocks between the barriers: always read it from L2
    volatile SelectState *st = a.st;
    const int tid = threadIdx.x, gtid = blockIdx.x * FUSED_THREADS + tid, gsize = gridDim.x * FUSED_THREADS;
    // written by an earlier launch only: every thread of every block reads the same value and leaves before
    // the first grid barrier
    if (a.stop && *a.stop) return;

    // ---- phase 0: state, histograms, candidate ids, optional rotation of the working set
    for (int i = gtid; i < lists * RADIX_BINS; i += gsize) a.hist[i] = 0;
    for (int i = gtid; i < lists * a.cap; i += gsize) a.cand_id[i] = -1;
    if (blockIdx.x == 0) {
        if (tid < lists) {
            st[tid].prefix_hi = 0; st[tid].prefix_lo = 0; st[tid].k_rem = a.want; st[tid].take_all = 0;
            st[tid].count = 0; st[tid].resolved = 0;
        }
        if (tid == 0) *a.ticket = 0;
        if (a.shift_ids && tid < a.shift_q) {
            const int leaving = a.shift_ids[tid], staying = a.shift_ids[a.shift_q + tid];
            if (leaving >= 0) a.shift_flags[leaving] = 0;
            if (staying >= 0) a.shift_flags[staying] = 1;
            a.shift_ids[tid] = staying;
        }
    }
    grid.sync();

    // ---- radix passes: one sweep each; the last block to finish its sweep picks the digits
    for (int pass = 0; pass < RADIX_PASSES; ++pass) {
        const int shift = 96 - RADIX_BITS * (pass + 1);
        unsigned active = 0;
        key96_t prefix[MAX_LISTS];
#pragma unroll
        for (int l = 0; l < MAX_LISTS; ++l) {
            prefix[l] = 0;
            if (l < lists && !st[l].take_all && !st[l].resolved) {
                active |= 1u << l;
                prefix[l] = ((key96_t) st[l].prefix_hi << 32) | st[l].prefix_lo;
            }
        }
        if (!active) break;                      // the same for every block: the state was final before the barrier
        for (int b = tid; b < lists * RADIX_BINS; b += FUSED_THREADS) sh[b] = 0;
        __syncthreads();
        for (int j = gtid; j < a.n; j += gsize) {
            if (a.in_ws && a.in_ws[j]) continue;
            const double al = a.alpha[j], fj = a.f[j];
            const int yj = a.y[j];
#pragma unroll
            for (int l = 0; l < MAX_LISTS; ++l) {
                if (!((active >> l) & 1u)) continue;
                if (!in_list(a.solver_kind, l, al, yj, a.Cp, a.Cn)) continue;
                const key96_t k = make_key(list_ascending(a.solver_kind, l), fj, (unsigned) j);
                if (pass > 0 && (k >> (shift + RADIX_BITS)) != (prefix[l] >> (shift + RADIX_BITS))) continue;
                const int bin = l * RADIX_BINS + ((int) (k >> shift) & (RADIX_BINS - 1));
                if (pass == 0) {
                    const unsigned peers = __match_any_sync(__activemask(), bin);
                    if ((int) (tid & 31) == __ffs(peers) - 1) atomicAdd(&sh[bin], __popc(peers));
                } else {
                    atomicAdd(&sh[bin], 1);
                }
            }
        }
        __syncthreads();
        for (int b = tid; b < lists * RADIX_BINS; b += FUSED_THREADS)
            if (sh[b]) atomicAdd(&a.hist[b], sh[b]);
        __threadfence();
        __syncthreads();
        if (tid == 0) is_last = (atomicAdd(a.ticket, 1) == (int) gridDim.x - 1);
        __syncthreads();
        if (is_last) {
            __threadfence();
            // All lists at once: threads 256 l .. 256 l + 255 own list l, 16 consecutive bins each. Exclusive scan of the
            // per-thread sums inside the list: warp shuffles, then the list's eight warp totals through shared memory.
            const int l = tid >> 8, t8 = tid & 255, lane = tid & 31;
            const bool mine = l < lists && ((active >> l) & 1u);
            int local[16], sum = 0;
            int *h = a.hist + l * RADIX_BINS + t8 * 16;
            if (mine) {
#pragma unroll
                for (int b4 = 0; b4 < 16; b4 += 4) {
                    const int4 v = __ldcg(reinterpret_cast<const int4 *>(h + b4));
                    local[b4] = v.x; local[b4 + 1] = v.y; local[b4 + 2] = v.z; local[b4 + 3] = v.w;
                    sum += v.x + v.y + v.z + v.w;
                }
            }
            int inc = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += v; }
            if (lane == 31) scan[tid >> 5] = inc;              // 32 warp totals: 8 per list
            __syncthreads();
            if (mine) {
                int before = inc - sum, total = 0;
                for (int w = 0; w < 8; ++w) {
                    const int v = scan[(l << 3) + w];
                    if (w < (t8 >> 5)) before += v;
                    total += v;
                }
                const int k_rem = st[l].k_rem;
                if (total < k_rem) {
                    if (t8 == 0) st[l].take_all = 1;   // can only happen in pass 0
                } else if (before < k_rem && k_rem <= before + sum) {
                    int run = before;
#pragma unroll
                    for (int b = 0; b < 16; ++b) {
                        if (run < k_rem && k_rem <= run + local[b]) {
                            key96_t p = prefix[l] | ((key96_t) (t8 * 16 + b) << shift);
                            const int k_new = k_rem - run;
                            if (shift > 0 && (a.want - k_new) + local[b] <= a.cap) {
                                p |= ((key96_t) 1 << shift) - 1;
                                st[l].resolved = 1;
                            }
                            st[l].prefix_hi = (unsigned long long) (p >> 32);
                            st[l].prefix_lo = (unsigned int) p;
                            st[l].k_rem = k_new;
                        }
                        run += local[b];
                    }
                }
#pragma unroll
                for (int b4 = 0; b4 < 16; b4 += 4) *reinterpret_cast<int4 *>(h + b4) = make_int4(0, 0, 0, 0);
            }
            __syncthreads();
            if (tid == 0) *a.ticket = 0;
            __threadfence();
        }
        grid.sync();
    }

    // ---- compaction of the candidates
    key96_t threshold[MAX_LISTS];
    bool take_all[MAX_LISTS];
#pragma unroll
    for (int l = 0; l < MAX_LISTS; ++l) {
        take_all[l] = l < lists ? st[l].take_all != 0 : true;
        threshold[l] = l < lists ? ((key96_t) st[l].prefix_hi << 32) | st[l].prefix_lo : 0;
    }
    for (int j0 = gtid - (tid & 31); j0 < a.n; j0 += gsize) {          // whole warps enter every round (ballots below)
        const int j = j0 + (tid & 31);
        const bool live = j < a.n && !(a.in_ws && a.in_ws[j]);
        const double al = live ? a.alpha[j] : 0.0, fj = live ? a.f[j] : 0.0;
        const int yj = live ? a.y[j] : 0;
        unsigned hit = 0;
#pragma unroll
        for (int l = 0; l < MAX_LISTS; ++l) {
            if (l >= lists || !live) continue;
            if (!in_list(a.solver_kind, l, al, yj, a.Cp, a.Cn)) continue;
            if (!take_all[l]) {
                const key96_t thr = threshold[l];
                if (make_key(list_ascending(a.solver_kind, l), fj, (unsigned) j) > thr) continue;
            }
            hit |= 1u << l;
        }
        // one atomic per warp and list instead of one per candidate
#pragma unroll
        for (int l = 0; l < MAX_LISTS; ++l) {
            if (l >= lists) continue;
            const unsigned peers = __ballot_sync(0xffffffffu, (hit >> l) & 1u);
            if (!peers) continue;
            int base = 0;
            if ((tid & 31) == __ffs(peers) - 1) base = atomicAdd(&a.st[l].count, __popc(peers));
            base = __shfl_sync(0xffffffffu, base, __ffs(peers) - 1);
            if ((hit >> l) & 1u) {
                const int pos = base + __popc(peers & ((1u << (tid & 31)) - 1));
                if (pos < a.cap) { a.cand_f[(size_t) l * a.cap + pos] = fj; a.cand_id[(size_t) l * a.cap + pos] = j + a.id_offset; }
            }
        }
    }
    if (a.mode == FUSED_CANDIDATES) return;
    __threadfence();
    grid.sync();
    // ---- the candidates are few: one block merges them / one block per list sorts them
    if (a.mode == FUSED_MERGE) {
        if (blockIdx.x == 0) merge_lists(a.solver_kind, a.cand_f, a.cand_id, a.cap, a.want, a.out_ids, a.out_count, 0, fused_smem);
    } else if ((int) blockIdx.x < lists) {
        sort_list(a.solver_kind, blockIdx.x, a.cand_f, a.cand_id, a.cap, a.sorted_f, a.sorted_id, a.want, fused_smem);
    }
}

static size_t merge_smem_bytes(int len) {
    int P = 1;
    while (P < len) P <<= 1;
    // keys of one list, or of all lists side by side where merge_lists sorts them together
    const size_t keys = (size_t) P * 12 * (P <= MERGE_JOINT_MAX ? MAX_LISTS : 1);
    return keys + (size_t) MAX_LISTS * MERGE_MAX_WANT * (4 + 2 + 1) + (size_t) HASH_SLOTS * 6 + 64;
}

// =================================================================================================
// Local SMO (one CTA per working set)
// =================================================================================================
// threads per local solver: 512 (two slots each) for a working set of 1,024 - measured 1.96 us per iteration
// against 2.14 with 256 threads and 2.10 with 1,024 -, 256 for smaller working sets
constexpr int SMO_THREADS_MAX = 512, SMO_WARPS_MAX = SMO_THREADS_MAX / 32;
constexpr unsigned long long KEY_POS_INF = 0xfff0000000000000ull;   // ordered_key(+inf)
constexpr int NO_SLOT = 0x7fffffff;

struct RedBuf {                     // per-warp partial results of up to four simultaneous reductions
    unsigned long long key[4][SMO_WARPS_MAX];
    int slot[4][SMO_WARPS_MAX];
};

// Block-wide argmin of R (key, slot) pairs: one __syncthreads, result in every thread.
template <int R, int SMO_WARPS>
__device__ __forceinline__ void block_argmin(RedBuf &buf, unsigned long long (&key)[R], int (&slot)[R]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        warp_argmin_u64(key[r], slot[r]);
        if (lane == 0) { buf.key[r][warp] = key[r]; buf.slot[r][warp] = slot[r]; }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
        unsigned long long k = lane < SMO_WARPS ? buf.key[r][lane] : ~0ull;
        int s = lane < SMO_WARPS ? buf.slot[r][lane] : NO_SLOT;
        warp_argmin_u64(k, s);
        key[r] = k; slot[r] = s;
    }
}

// Local solver. Slot t of the working set is owned by thread t % 256 (register copies of f, alpha,
// y, diag); mirrors of f / alpha / y / diag in shared memory serve the few values every thread
// needs from the selected pair. kww is the ws x ws kernel block, so row loads are coalesced.
// NU = false: c_smo_solve_kernel semantics of the CPU backend (smo_kernel.cpp:12-125), ties to the
// lowest slot. NU = true: nu_smo_solve_kernel semantics of the CUDA backend
// (smo_kernel.cu:118-252): bound held in float, float arithmetic in the curvature term.
template <bool NU, int SLOTS, int SMO_THREADS>
__global__ void __launch_bounds__(SMO_THREADS)
local_smo_kernel(int ws, const float *__restrict__ kww, const float *__restrict__ diag_ws,
                 const int *__restrict__ y_ws, const double *__restrict__ f_ws, double *__restrict__ alpha_ws,
                 double *__restrict__ alpha_diff, double Cp_in, double Cn_in, double eps, int max_iter,
                 double *__restrict__ diff, const int *__restrict__ ids, double *__restrict__ alpha_global,
                 const int *__restrict__ stop) {
    if (stop && *stop) {            // queued past the end of a solve: no step, so the f update that follows adds zero
        for (int t = threadIdx.x; t < ws; t += SMO_THREADS) alpha_diff[t] = 0;
        return;
    }
    __shared__ RedBuf red[2];
    __shared__ double f_sm[1024], a_sm[1024];
    __shared__ float kd_sm[1024];
    __shared__ int y_sm[1024];
    const double Cp = NU ? (double) (float) Cp_in : Cp_in;
    const double Cn = NU ? Cp : Cn_in;
    const int tid = threadIdx.x;
    double f[SLOTS], a[SLOTS], aold[SLOTS];
    int y[SLOTS];
    float kd[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const int t = tid + s * SMO_THREADS;
        if (t < ws) {
            f[s] = f_ws[t]; a[s] = aold[s] = alpha_ws[t]; y[s] = y_ws[t]; kd[s] = diag_ws[t];
            f_sm[t] = f[s]; a_sm[t] = a[s]; y_sm[t] = y[s]; kd_sm[t] = kd[s];
        } else { f[s] = 0; a[s] = aold[s] = 0; y[s] = 0; kd[s] = 0; }   // y = 0: member of no set
    }
    // Membership of I_up / I_low only changes for the two slots a step moves, so it is kept in registers and
    // recomputed for those two instead of for every slot in every selection
    bool in_up[SLOTS], in_low[SLOTS];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        in_up[s] = in_I_up(a[s], y[s], Cp, Cn);
        in_low[s] = in_I_low(a[s], y[s], Cp, Cn);
    }
    __syncthreads();
    double local_eps = 0;
    int it = 0;
    for (;;) {
        // ---- first-order selection --------------------------------------------------------
        constexpr int R1 = NU ? 4 : 2;
        unsigned long long key[R1];
        int slot[R1];
#pragma unroll
        for (int r = 0; r < R1; ++r) { key[r] = KEY_POS_INF; slot[r] = NO_SLOT; }
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int t = tid + s * SMO_THREADS;
            const unsigned long long kf = ordered_key(f[s]), knf = ordered_key(-f[s]);
            if (!NU) {
                if (in_up[s] && kf < key[0]) { key[0] = kf; slot[0] = t; }
                if (in_low[s] && knf < key[1]) { key[1] = knf; slot[1] = t; }
            } else {
                // the four lists are I_up and I_low split by class (Cn = Cp here)
                if (y[s] > 0 && in_up[s] && kf < key[0]) { key[0] = kf; slot[0] = t; }       // up, +:  a < C
                if (y[s] < 0 && in_up[s] && kf < key[1]) { key[1] = kf; slot[1] = t; }       // up, -:  a > 0
                if (y[s] > 0 && in_low[s] && knf < key[2]) { key[2] = knf; slot[2] = t; }    // low, +: a > 0
                if (y[s] < 0 && in_low[s] && knf < key[3]) { key[3] = knf; slot[3] = t; }    // low, -: a < C
            }
        }
        block_argmin<R1, SMO_THREADS / 32>(red[0], key, slot);
        // mirrors written only now: every thread has finished reading them for the last step
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int t = tid + s * SMO_THREADS;
            if (t < ws) { f_sm[t] = f[s]; a_sm[t] = a[s]; }
        }
        const int i0 = slot[0] == NO_SLOT ? 0 : slot[0];
        const int i1 = NU ? (slot[1] == NO_SLOT ? 0 : slot[1]) : 0;
        const double up0 = key_to_double(key[0]);
        const double up1 = NU ? key_to_double(key[1]) : 0.0;
        float kI0[SLOTS], kI1[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int t = tid + s * SMO_THREADS;
            kI0[s] = t < ws ? __ldg(kww + (size_t) i0 * ws + t) : 0.0f;
            kI1[s] = (NU && t < ws) ? __ldg(kww + (size_t) i1 * ws + t) : 0.0f;
        }
        double local_diff;
        if (!NU) local_diff = -key_to_double(key[1]) - up0;
        else local_diff = fmax(-key_to_double(key[2]) - up0, -key_to_double(key[3]) - up1);
        if (it == 0) {
            local_eps = NU ? fmax(eps, 0.1 * local_diff) : fmax(eps, (double) 0.1f * local_diff);
            if (tid == 0) diff[0] = local_diff;
        }
        if (it > max_iter || local_diff < local_eps) break;

        // ---- second-order selection ---------------------------------------------------------
        constexpr int R2 = NU ? 2 : 1;
        unsigned long long key2[R2];
        int slot2[R2];
#pragma unroll
        for (int r = 0; r < R2; ++r) { key2[r] = KEY_POS_INF; slot2[r] = NO_SLOT; }
        const float kd_i0 = kd_sm[i0], kd_i1 = NU ? kd_sm[i1] : 0.0f;
        if (!NU) {
            // The exact quotient -b^2 / a costs a double-precision division per slot, and only the thread's best
            // slot matters. An FP32 estimate of b^2 / a (relative error below 5e-7: two roundings to FP32, a
            // product, a 2-ulp division) first rules out every slot whose estimate is more than 8e-6 below the
            // thread's largest: its exact quotient is smaller by more than any rounding, so it can neither win nor
            // tie. What is left - almost always one slot - is divided exactly. Estimates outside the range
            // where the error bound holds send all of the thread's candidates to the exact path.
            bool cnd[SLOTS];
            double aIJ[SLOTS], bIJ[SLOTS];
            float q32[SLOTS];
            float m = -1.0f;
            bool trust = true;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                cnd[s] = -up0 > -f[s] && in_low[s];
                aIJ[s] = (double) (kd_i0 + kd[s]) - 2.0 * (double) kI0[s];
                bIJ[s] = -up0 + f[s];
                const float b32 = (float) bIJ[s], a32 = (float) aIJ[s];
                q32[s] = __fdividef(b32 * b32, a32);
                trust = trust && (!cnd[s] || (b32 > 1e-15f && b32 < 1e15f && a32 > 1e-30f && a32 < 1e30f));
                if (cnd[s]) m = fmaxf(m, q32[s]);
            }
            const float thr = m * (1.0f - 8e-6f);
            // the first slot that holds the largest estimate, divided without a branch
            int pick = SLOTS;
            double pa = 1.0, pb = 0.0;
#pragma unroll
            for (int s = SLOTS - 1; s >= 0; --s)
                if (cnd[s] && q32[s] == m) { pick = s; pa = aIJ[s]; pb = bIJ[s]; }
            if (pick < SLOTS) {
                key2[0] = ordered_key(-pb * pb / pa);
                slot2[0] = tid + pick * SMO_THREADS;
            }
            // any other slot the estimate cannot rule out: exact, ties to the lower slot as in a pass in slot order
            bool more = false;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) more = more || (cnd[s] && s != pick && (!trust || q32[s] >= thr));
            if (more) {
#pragma unroll
                for (int s = 0; s < SLOTS; ++s) {
                    if (cnd[s] && s != pick && (!trust || q32[s] >= thr)) {
                        const int t = tid + s * SMO_THREADS;
                        const unsigned long long k = ordered_key(-bIJ[s] * bIJ[s] / aIJ[s]);
                        if (k < key2[0] || (k == key2[0] && t < slot2[0])) { key2[0] = k; slot2[0] = t; }
                    }
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int t = tid + s * SMO_THREADS;
                // every slot computes its quotients, candidates or not (the others divide by one and are
                // discarded): the divisions of a thread's slots then overlap instead of one divergent branch each
                const bool c0 = -up0 > -f[s] && y[s] > 0 && in_low[s];
                const bool c1 = -up1 > -f[s] && y[s] < 0 && in_low[s];
                const double a0 = (double) (kd_i0 + kd[s] - 2 * kI0[s]), a1 = (double) (kd_i1 + kd[s] - 2 * kI1[s]);
                const double b0 = -up0 + f[s], b1 = -up1 + f[s];
                const double v0 = -b0 * b0 / (c0 ? a0 : 1.0), v1 = -b1 * b1 / (c1 ? a1 : 1.0);
                const unsigned long long k0 = ordered_key(v0), k1 = ordered_key(v1);
                if (c0 && k0 < key2[0]) { key2[0] = k0; slot2[0] = t; }
                if (c1 && k1 < key2[1]) { key2[1] = k1; slot2[1] = t; }
            }
        }
        block_argmin<R2, SMO_THREADS / 32>(red[1], key2, slot2);
        int i, j2;
        double up;
        bool use1 = false;
        if (!NU) { i = i0; j2 = slot2[0] == NO_SLOT ? 0 : slot2[0]; up = up0; }
        else {
            // the positive-class pair wins only if its value is strictly smaller (smo_kernel.cu:220-233)
            if (key_to_double(key2[0]) < key_to_double(key2[1])) { i = i0; j2 = slot2[0] == NO_SLOT ? 0 : slot2[0]; up = up0; }
            else { i = i1; j2 = slot2[1] == NO_SLOT ? 0 : slot2[1]; up = up1; use1 = true; }
        }
        // ---- step length, computed redundantly by every thread ---------------------------------
        const double ai = a_sm[i], aj = a_sm[j2], fj = f_sm[j2];
        const int yi = y_sm[i], yj = y_sm[j2];
        const float kij = __ldg(kww + (size_t) i * ws + j2);
        float kJ[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int t = tid + s * SMO_THREADS;
            kJ[s] = t < ws ? __ldg(kww + (size_t) j2 * ws + t) : 0.0f;
        }
        const double alpha_i_diff = yi > 0 ? Cp - ai : ai;
        const double curv = NU ? (double) (kd_sm[i] + kd_sm[j2] - 2 * kij)
                               : (double) (kd_sm[i] + kd_sm[j2]) - 2.0 * (double) kij;
        const double alpha_j_diff = fmin(yj > 0 ? aj : Cn - aj, (-up + fj) / curv);
        const double l = fmin(alpha_i_diff, alpha_j_diff);
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int t = tid + s * SMO_THREADS;
            if (t == i) a[s] += l * yi;
            if (t == j2) a[s] -= l * yj;
            if (t == i || t == j2) {
                in_up[s] = in_I_up(a[s], y[s], Cp, Cn);
                in_low[s] = in_I_low(a[s], y[s], Cp, Cn);
            }
            if (t < ws) {
                const float kI = use1 ? kI1[s] : kI0[s];
                if (NU) f[s] -= l * (double) (kJ[s] - kI);
                else f[s] -= l * ((double) kJ[s] - (double) kI);
            }
        }
        ++it;
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const int t = tid + s * SMO_THREADS;
        if (t < ws) {
            alpha_ws[t] = a[s];
            alpha_diff[t] = -(a[s] - aold[s]) * y[s];
            if (alpha_global && ids[t] >= 0) alpha_global[ids[t]] = a[s];
        }
    }
    if (tid == 0) diff[1] = it;
}

// ---- gather of the working set's block and vectors ---------------------------------------------
// Logical slot t of the working set lives in physical row phys(t) of the row buffer (the two
// halves of the buffer swap roles every outer iteration instead of being copied).
__device__ __forceinline__ int phys_row(int t, int q, int first_half_phys) {
    return t < q ? first_half_phys * q + t : (1 - first_half_phys) * q + (t - q);
}

__global__ void gather_ws_kernel(int ws, int q, int first_half_phys, const int *__restrict__ ids,
                                 const float *__restrict__ rows, long long ld, const float *__restrict__ diag,
                                 const int *__restrict__ y, const double *__restrict__ f,
                                 const double *__restrict__ alpha, float *__restrict__ kww,
                                 float *__restrict__ diag_ws, int *__restrict__ y_ws, double *__restrict__ f_ws,
                                 double *__restrict__ alpha_ws, int block_rows, const int *__restrict__ row_slot) {
    const int a = blockIdx.x;                      // logical slot of the row
    // rows >= block_rows of the block are written by someone else (the overlapped iteration computes them
    // directly); the slot vectors are gathered for every slot
    // a slot without an instance (id -1: fewer eligible instances than slots) is inert: y = 0 puts it in no set
    if (a < block_rows) {
        const float *row = rows + (size_t) (row_slot ? row_slot[a] : phys_row(a, q, first_half_phys)) * ld;
        for (int b = threadIdx.x; b < ws; b += blockDim.x) {
            const int id = ids[b];
            kww[(size_t) a * ws + b] = id >= 0 ? row[id] : 0.0f;
        }
    }
    if (threadIdx.x == 0) {
        const int id = ids[a];
        if (id >= 0) { diag_ws[a] = diag[id]; y_ws[a] = y[id]; f_ws[a] = f[id]; alpha_ws[a] = alpha[id]; }
        else { diag_ws[a] = 1.0f; y_ws[a] = 0; f_ws[a] = 0.0; alpha_ws[a] = 0.0; }
    }
}

// =================================================================================================
// Kernel-row cache: least-recently-used rows kept in HBM
// =================================================================================================
// The reference keeps only the previous iteration's q rows (csmosolver.cpp:69,75). Here the row buffer has
// room for `cap` rows (as many as the memory budget allows, at least ws + q). A directory on the device maps
// instance -> row (slot_of), row -> instance (inst_of) and row -> outer iteration of its last use (stamp).
// After every selection one block looks the new members up: a hit only points the member's slot at the cached
// row; the misses are compacted into the list the kernel-row engine then computes, and each gets the row of a
// victim - the rows with the oldest stamps that do not belong to the current working set, found with a
// histogram over the stamps; ties go to the lower row number, so the choice does not depend on thread timing.
// Everything stays on the device: the engine reads the number of misses from memory.
constexpr int CACHE_THREADS = 1024, CACHE_BINS = 2048;
enum { CACHE_N_MISS = 0, CACHE_HITS = 1, CACHE_MISSES = 2, CACHE_BLOCKS = 3, CACHE_BLOCKS_SAVED = 4,
       CACHE_NEXT_FREE = 5,         // rows [0, next_free) have been handed out; the rest never held a row
       CACHE_CTRS = 8 };

__device__ __forceinline__ int cache_bin(int stamp, int now) {
    // older -> smaller bin; never-used rows (stamp 0) are the oldest; rows used in this iteration are not candidates
    if (stamp <= 0) return 0;
    const int age = now - stamp;
    return age >= CACHE_BINS - 1 ? 0 : CACHE_BINS - 1 - age;
}

__global__ void __launch_bounds__(CACHE_THREADS, 1)
cache_assign_kernel(const int *__restrict__ ids, int t0, int n_new, int now, int *__restrict__ slot_of,
                    int *__restrict__ inst_of, int *__restrict__ stamp, int cap, int *__restrict__ row_slot,
                    int *__restrict__ miss_ids, int *__restrict__ miss_slot, int *__restrict__ victims,
                    long long *__restrict__ ctr, int row_block, const int *__restrict__ stop) {
    if (stop && *stop) {            // queued past the end of a solve: no member changes, no row to compute
        if (threadIdx.x == 0) reinterpret_cast<int *>(ctr)[0] = 0;
        return;
    }
    __shared__ int hist[CACHE_BINS];
    __shared__ int miss_t[CACHE_THREADS];
    __shared__ int wsum[32], wpre_b[32], wpre_sel[32];
    __shared__ int n_miss_s, thr_bin, need_s, n_hit_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the members that stay move to the front; their rows are in use now
    int keep = 0;
    if (tid < t0) keep = row_slot[t0 + tid];
    for (int b = tid; b < CACHE_BINS; b += CACHE_THREADS) hist[b] = 0;
    if (tid == 0) { n_miss_s = 0; n_hit_s = 0; }
    __syncthreads();
    if (tid < t0) { row_slot[tid] = keep; if (ids[tid] >= 0) stamp[keep] = now; }
    // look the new members up; misses are compacted in member order
    int id = -1, s = -1;
    if (tid < n_new) {
        id = ids[t0 + tid];
        s = id >= 0 ? slot_of[id] : -1;
        if (id < 0) row_slot[t0 + tid] = 0;            // an empty working-set slot is inert: any row will do
        else if (s >= 0) { row_slot[t0 + tid] = s; stamp[s] = now; }
    }
    const bool miss = tid < n_new && id >= 0 && s < 0;
    const unsigned mb = __ballot_sync(0xffffffffu, miss);
    if (lane == 0) wsum[warp] = __popc(mb);
    const unsigned hb = __ballot_sync(0xffffffffu, tid < n_new && id >= 0 && s >= 0);
    if (lane == 0 && hb) atomicAdd(&n_hit_s, __popc(hb));
    __syncthreads();
    if (warp == 0) {
        const int v = wsum[lane];
        int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += a; }
        wsum[lane] = inc - v;
        if (lane == 31) n_miss_s = inc;
    }
    __syncthreads();
    if (miss) miss_t[wsum[warp] + __popc(mb & ((1u << lane) - 1))] = tid;
    const int n_miss = n_miss_s;
    // (the stamps written above must be visible to the sweeps below)
    __threadfence_block();
    __syncthreads();
    // While rows that never held anything are left, the misses take the lowest of them - the rows the sweeps
    // below would pick (stamp 0 is the oldest, ties go to the lower row) without sweeping the stamps.
    __shared__ long long next_free_s;
    if (tid == 0) next_free_s = ctr[CACHE_NEXT_FREE];
    __syncthreads();
    const long long next_free = next_free_s;
    const bool fresh = next_free + n_miss <= cap;
    if (n_miss > 0 && fresh) {
        if (tid < n_miss) victims[tid] = (int) next_free + tid;
        __threadfence_block();
        __syncthreads();
    } else if (n_miss > 0) {
        // histogram of the candidates' stamps
        for (int r = tid; r < cap; r += CACHE_THREADS) {
            const int st = stamp[r];
            if (st != now) atomicAdd(&hist[cache_bin(st, now)], 1);
        }
        __syncthreads();
        // threshold bin: the n_miss oldest rows are all rows of the bins below it and `need` rows of the bin itself
        if (warp == 0) {
            int run = 0, found = 0;
            for (int b0 = 0; b0 < CACHE_BINS && !found; b0 += 32) {
                const int v = hist[b0 + lane];
                int inc = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += a; }
                const unsigned reach = __ballot_sync(0xffffffffu, run + inc >= n_miss);
                if (reach) {
                    const int l = __ffs(reach) - 1;
                    const int before = run + __shfl_sync(0xffffffffu, inc - v, l);
                    if (lane == 0) { thr_bin = b0 + l; need_s = n_miss - before; }
                    found = 1;
                }
                run += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (!found && lane == 0) { thr_bin = CACHE_BINS; need_s = 0; }     // cannot happen: cap >= ws + q
        }
        __syncthreads();
        const int B = thr_bin, need = need_s;
        // ordered choice: every warp owns a contiguous range of rows
        const int per = (cap + 31) / 32;
        const int r0 = warp * per, r1 = min(cap, r0 + per);
        int cnt_b = 0, cnt_l = 0;
        for (int r = r0 + lane; r - lane < r1; r += 32) {
            const int st = r < r1 ? stamp[r] : now;
            const int bin = st != now ? cache_bin(st, now) : CACHE_BINS;
            cnt_b += __popc(__ballot_sync(0xffffffffu, bin == B));
            cnt_l += __popc(__ballot_sync(0xffffffffu, bin < B));
        }
        if (lane == 0) { wpre_b[warp] = cnt_b; wpre_sel[warp] = cnt_l; }
        __syncthreads();
        if (warp == 0) {
            const int vb = wpre_b[lane], vl = wpre_sel[lane];
            int ib = vb;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, ib, o); if (lane >= o) ib += a; }
            const int pre_b = ib - vb;
            const int take_b = max(0, min(vb, need - pre_b));
            int isel = vl + take_b;
            const int vsel = isel;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, isel, o); if (lane >= o) isel += a; }
            wpre_b[lane] = pre_b;
            wpre_sel[lane] = isel - vsel;
        }
        __syncthreads();
        int run_b = wpre_b[warp], pos = wpre_sel[warp];
        for (int r = r0 + lane; r - lane < r1; r += 32) {
            const int st = r < r1 ? stamp[r] : now;
            const int bin = st != now ? cache_bin(st, now) : CACHE_BINS;
            const unsigned bb = __ballot_sync(0xffffffffu, bin == B);
            const int rank_b = run_b + __popc(bb & ((1u << lane) - 1));
            const bool sel = bin < B || (bin == B && rank_b < need);
            const unsigned sb = __ballot_sync(0xffffffffu, sel);
            if (sel) victims[pos + __popc(sb & ((1u << lane) - 1))] = r;
            run_b += __popc(bb);
            pos += __popc(sb);
        }
        __threadfence_block();
        __syncthreads();
    }
    if (n_miss > 0) {
        // the misses take the victims' rows
        if (tid < n_miss) {
            const int t = miss_t[tid];
            const int mid = ids[t0 + t];
            const int r = victims[tid];
            const int old = inst_of[r];
            if (old >= 0) slot_of[old] = -1;
            inst_of[r] = mid;
            slot_of[mid] = r;
            stamp[r] = now;
            row_slot[t0 + t] = r;
            miss_ids[tid] = mid;
            miss_slot[tid] = r;
        }
    }
    if (tid == 0) {
        reinterpret_cast<int *>(ctr)[0] = n_miss;                 // CACHE_N_MISS, read by the engines as an int
        ctr[CACHE_HITS] += n_hit_s;
        ctr[CACHE_MISSES] += n_miss;
        ctr[CACHE_BLOCKS] += (n_new + row_block - 1) / row_block;
        ctr[CACHE_BLOCKS_SAVED] += (n_new + row_block - 1) / row_block - (n_miss + row_block - 1) / row_block;
        ctr[CACHE_NEXT_FREE] = fresh ? next_free + n_miss : (long long) cap;
    }
}

// ---- end-of-iteration bookkeeping on the device ----------------------------------------------------
// The reference decides after every outer iteration, on the host, whether to go on (csmosolver.cpp:83-111).
// Here one thread applies the same rules to the same doubles on the device, so the host can queue several
// iterations and read the outcome once: every kernel of a queued iteration looks at `stop` first and does
// nothing once it is set.
struct SolverCtl {
    int stop;                       // first member: kernels take a pointer to it
    int done;                       // the reference's own termination rules fired
    int iter, same_cnt, swap_cnt;
    int short_got, short_wanted;    // a selection that could not fill its slots (got < wanted)
    int engine_status;              // non-zero: a bounded wait of the kernel-row engine ran out
    double prev, last, second_last, diff0;
    long long local_iter;
    long long ctr[CACHE_CTRS];      // cache counters as of the last iteration that ran
};
static_assert(offsetof(SolverCtl, stop) == 0, "kernels read the stop flag through a pointer to the struct");

__global__ void solver_status_kernel(SolverCtl *c, const double *__restrict__ diff, const int *__restrict__ got,
                                     int wanted, double eps, int max_iter, const long long *__restrict__ cache_ctr,
                                     const int *__restrict__ engine_status) {
    if (threadIdx.x != 0 || c->stop) return;
    const double d = diff[0];
    c->diff0 = d;
    c->local_iter += (long long) diff[1];
    // csmosolver.cpp:86-111
    if (fabs(d - c->prev) < eps * 0.001) c->same_cnt++;
    else { c->same_cnt = 0; c->prev = d; }
    if (fabs(d - c->second_last) < eps * 0.001) c->swap_cnt++;
    else c->swap_cnt = 0;
    c->second_last = c->last;
    c->last = d;
    int stop = 0;
    if ((c->same_cnt >= 10 && fabs(d - 2.0) > eps) || d < eps || (c->swap_cnt >= 10 && fabs(d - 2.0) > eps)) {
        c->done = 1;
        stop = 1;
    }
    c->iter++;
    if (max_iter != -1 && c->iter - 1 == max_iter) stop = 1;      // iteration cap (csmosolver.cpp:110)
    if (*got < wanted) { c->short_got = *got; c->short_wanted = wanted; stop = 1; }
    if (engine_status && *engine_status) { c->engine_status = *engine_status; stop = 1; }
    if (cache_ctr)
        for (int k = 0; k < CACHE_CTRS; ++k) c->ctr[k] = cache_ctr[k];
    c->stop = stop;
}

__global__ void fill_int_kernel(int *p, long long n, int v) {
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long) gridDim.x * blockDim.x) p[i] = v;
}

// =================================================================================================
// f update:  f[j] -= sum_t alpha_diff[t] * rows[phys(t)][j]   (smo_kernel.cu:289-310)
// =================================================================================================
// HBM-bound: every thread owns 4 consecutive columns and streams the rows whose alpha_diff is
// non-zero with 16-byte loads, 16 rows in flight.
__global__ void __launch_bounds__(128)
update_f_kernel(double *__restrict__ f, int n, const double *__restrict__ alpha_diff, int ws, int q,
                int first_half_phys, const float *__restrict__ rows, long long ld, int vec_ok, int t_begin,
                int t_end, int cols, const int *__restrict__ row_slot) {
    __shared__ double ad[1024];
    __shared__ int prow[1024];
    __shared__ int cnt;
    if (threadIdx.x == 0) cnt = 0;
    __syncthreads();
    // order-preserving compaction of the non-zero entries (one warp, ballot scan)
    if (threadIdx.x < 32) {
        int base = 0;
        // slots [t_begin, t_end) of the working set (t_begin a multiple of 32)
        for (int t0 = t_begin; t0 < t_end; t0 += 32) {
            const int t = t0 + threadIdx.x;
            const double dv = t < t_end ? alpha_diff[t] : 0.0;
            const unsigned m = __ballot_sync(0xffffffffu, dv != 0.0);
            if (dv != 0.0) {
                const int p = base + __popc(m & ((1u << threadIdx.x) - 1));
                ad[p] = dv;
                prow[p] = row_slot ? row_slot[t] : (q > 0 ? phys_row(t, q, first_half_phys) : t);
            }
            base += __popc(m);
        }
        if (threadIdx.x == 0) cnt = base;
    }
    __syncthreads();
    const int m = cnt;
    if (cols == 1) {
        // short shards: one column per thread, so that enough loads are in flight to cover the HBM latency
        // (same order of summation per column as the four-column form)
        const long long c = (long long) blockIdx.x * blockDim.x + threadIdx.x;
        if (c >= n) return;
        double s = 0;
        int r = 0;
        for (; r + 16 <= m; r += 16) {
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = __ldcs(rows + (size_t) prow[r + u] * ld + c);
#pragma unroll
            for (int u = 0; u < 16; ++u) s += ad[r + u] * v[u];
        }
        for (; r < m; ++r) s += ad[r] * __ldcs(rows + (size_t) prow[r] * ld + c);
        f[c] -= s;
        return;
    }
    const long long j = ((long long) blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (j >= n) return;
    double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    if (j + 3 < n && vec_ok) {
        int r = 0;
        for (; r + 16 <= m; r += 16) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = __ldcs(reinterpret_cast<const float4 *>(rows + (size_t) prow[r + u] * ld + j));
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const double dv = ad[r + u];
                s0 += dv * v[u].x; s1 += dv * v[u].y; s2 += dv * v[u].z; s3 += dv * v[u].w;
            }
        }
        for (; r < m; ++r) {
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(rows + (size_t) prow[r] * ld + j));
            const double dv = ad[r];
            s0 += dv * v.x; s1 += dv * v.y; s2 += dv * v.z; s3 += dv * v.w;
        }
        f[j] -= s0; f[j + 1] -= s1; f[j + 2] -= s2; f[j + 3] -= s3;
    } else {
        for (int c = 0; c < 4 && j + c < n; ++c) {
            double s = 0;
            for (int r = 0; r < m; ++r) s += ad[r] * rows[(size_t) prow[r] * ld + j + c];
            f[j + c] -= s;
        }
    }
}

// =================================================================================================
// rho / objective
// =================================================================================================
// out[0..12] = n_free(+), sum_free f(+), n_free(-), sum_free f(-), sum of the objective terms,
//              min f over I_up (+), max f over I_low (+), the same two for (-),
//              max f over I_up (+), min f over I_low (+), the same two for (-).
constexpr int RHO_VALS = 13;
__global__ void __launch_bounds__(1024)
rho_obj_kernel(int n, const double *__restrict__ f, const double *__restrict__ alpha, const int *__restrict__ y,
               double Cp, double Cn, double *__restrict__ out) {
    __shared__ double sh[32][RHO_VALS];
    double v[RHO_VALS] = {0, 0, 0, 0, 0, INFINITY, -INFINITY, INFINITY, -INFINITY, -INFINITY, INFINITY, -INFINITY,
                          INFINITY};
    for (int i = threadIdx.x; i < n; i += 1024) {
        const double a = alpha[i], fi = f[i];
        const int yi = y[i];
        v[4] += a - (fi + yi) * a * yi / 2;
        const bool up = in_I_up(a, yi, Cp, Cn), low = in_I_low(a, yi, Cp, Cn);
        if (yi > 0) {
            if (a > 0 && a < Cp) { v[0] += 1; v[1] += fi; }
            if (up) { v[5] = fmin(v[5], fi); v[9] = fmax(v[9], fi); }
            if (low) { v[6] = fmax(v[6], fi); v[10] = fmin(v[10], fi); }
        } else {
            if (a > 0 && a < Cn) { v[2] += 1; v[3] += fi; }
            if (up) { v[7] = fmin(v[7], fi); v[11] = fmax(v[11], fi); }
            if (low) { v[8] = fmax(v[8], fi); v[12] = fmin(v[12], fi); }
        }
    }
    auto combine = [](int k, double a, double b) -> double {
        if (k < 5) return a + b;
        const bool is_min = (k == 5 || k == 7 || k == 10 || k == 12);
        return is_min ? fmin(a, b) : fmax(a, b);
    };
    for (int o = 16; o; o >>= 1)
#pragma unroll
        for (int k = 0; k < RHO_VALS; ++k) v[k] = combine(k, v[k], __shfl_xor_sync(0xffffffffu, v[k], o));
    if ((threadIdx.x & 31) == 0)
        for (int k = 0; k < RHO_VALS; ++k) sh[threadIdx.x >> 5][k] = v[k];
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; ++w)
            for (int k = 0; k < RHO_VALS; ++k) sh[0][k] = combine(k, sh[0][k], sh[w][k]);
        for (int k = 0; k < RHO_VALS; ++k) out[k] = sh[0][k];
    }
}

__global__ void scale_kernel(double *a, int n, double r) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] /= r;
}

// =================================================================================================
// Column-sharded solver: per-rank device work of one outer iteration (the exchange steps between the
// phases belong to the caller)
// =================================================================================================

// all-gathered candidate lists [world][lists][want] -> [lists][world * want]
__global__ void shard_regroup_kernel(const double *__restrict__ gf, const int *__restrict__ gi, int world, int lists,
                                     int want, double *__restrict__ of, int *__restrict__ oi) {
    const int total = world * lists * want;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int r = e / (lists * want), rem = e - r * lists * want, l = rem / want, p = rem - l * want;
        const size_t o = (size_t) l * world * want + (size_t) r * want + p;
        of[o] = gf[e];
        oi[o] = gi[e];
    }
}

// Slots 0..q-1 <- slots q..ws-1 (global ids and per-member vectors); in-working-set flags of the owned
// instances: the old first half leaves, the old second half stays. One block, q <= 512.
__global__ void shard_shift_kernel(int *ids, int q, int lo, int hi, unsigned char *in_ws, float *m_sd,
                                   float *m_unscale, float *m_diag) {
    const int t = threadIdx.x;
    if (t < q) {
        const int leaving = ids[t], staying = ids[q + t];
        if (leaving >= lo && leaving < hi) in_ws[leaving - lo] = 0;
        if (staying >= lo && staying < hi) in_ws[staying - lo] = 1;
        ids[t] = staying;
        m_sd[t] = m_sd[q + t]; m_unscale[t] = m_unscale[q + t]; m_diag[t] = m_diag[q + t];
    }
}

// What this rank contributes to the exchange after the selection: for the n_new new members (slots slot0..)
// their feature row, self dot and diagonal (zeros if another rank owns them) -> crow[s][0..d), [dp], [dp+1]
// (row stride ldw = dp + 4, dp = round_up(d, 4)); for all ws members (y, f, alpha) -> cstate[slot][3].
// Summing the contributions of all ranks gives the values (adding zeros is exact).
__global__ void shard_contrib_kernel(const int *__restrict__ ids, int slot0, int n_new, int ws, int lo, int hi,
                                     const float *__restrict__ X, int ldx, int d, int dp, const float *__restrict__ sd,
                                     const float *__restrict__ diag, const int *__restrict__ y,
                                     const double *__restrict__ f, const double *__restrict__ alpha,
                                     float *__restrict__ crow, double *__restrict__ cstate) {
    const int b = blockIdx.x;
    if (b < n_new) {
        const int gid = ids[slot0 + b];
        const bool own = gid >= lo && gid < hi;
        float *dst = crow + (size_t) b * (dp + 4);
        const float *src = own ? X + (size_t) (gid - lo) * ldx : nullptr;
        for (int k = threadIdx.x; k < dp + 4; k += blockDim.x) {
            float v = 0.0f;
            if (own) {
                if (k < d) v = src[k];
                else if (k == dp) v = sd[gid - lo];
                else if (k == dp + 1) v = diag[gid - lo];
            }
            dst[k] = v;
        }
    } else {
        for (int t = (b - n_new) * blockDim.x + threadIdx.x; t < ws; t += (gridDim.x - n_new) * blockDim.x) {
            const int gid = ids[t];
            const bool own = gid >= lo && gid < hi;
            cstate[3 * t] = own ? (double) y[gid - lo] : 0.0;
            cstate[3 * t + 1] = own ? f[gid - lo] : 0.0;
            cstate[3 * t + 2] = own ? alpha[gid - lo] : 0.0;
        }
    }
}

// After the exchange: member vectors of the new slots out of the row buffer, solver inputs out of the state.
__global__ void shard_unpack_kernel(const float *__restrict__ crow, int slot0, int n_new, int dp, int ws,
                                    const double *__restrict__ cstate, float *__restrict__ m_sd,
                                    float *__restrict__ m_diag, int *__restrict__ y_ws, double *__restrict__ f_ws,
                                    double *__restrict__ a_ws) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n_new) {
        m_sd[slot0 + t] = crow[(size_t) t * (dp + 4) + dp];
        m_diag[slot0 + t] = crow[(size_t) t * (dp + 4) + dp + 1];
    }
    if (t < ws) {
        y_ws[t] = (int) cstate[3 * t];
        f_ws[t] = cstate[3 * t + 1];
        a_ws[t] = cstate[3 * t + 2];
    }
}

// alpha of the owned members back into the rank's slice
__global__ void shard_scatter_kernel(const int *__restrict__ ids, int ws, int lo, int hi,
                                     const double *__restrict__ a_ws, double *__restrict__ alpha) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < ws) {
        const int gid = ids[t];
        if (gid >= lo && gid < hi) alpha[gid - lo] = a_ws[t];
    }
}

// =================================================================================================
// host side
// =================================================================================================
// f update: four columns per thread (16-byte loads) for long column ranges, one for short ones
static inline int update_f_cols(long long n) { return n >= 300000 ? 4 : 1; }
static inline int update_f_grid(long long n) { return ceil_div(n, 128 * update_f_cols(n)); }
static inline int rows_vec_ok(const float *rows, long long ld) {
    return (((uintptr_t) rows & 15) == 0 && (ld & 3) == 0) ? 1 : 0;
}

static tsvm_status launch_local_smo(int solver_kind, int ws, const float *kww, const float *diag_ws, const int *y_ws,
                                    const double *f_ws, double *alpha_ws, double *alpha_diff, double Cp, double Cn,
                                    double eps, int max_iter, double *diff, const int *ids, double *alpha_global,
                                    cudaStream_t st, const int *stop = nullptr) {
    const bool nu = solver_kind != TSVM_SOLVER_C;
#define SMO_CASE(NU, S, T)                                                                                     \
    TSVM_LAUNCH((local_smo_kernel<NU, S, T>), 1, T, 0, st, ws, kww, diag_ws, y_ws, f_ws, alpha_ws,             \
                alpha_diff, Cp, Cn, eps, max_iter, diff, ids, alpha_global, stop)
    if (!nu) {
        if (ws <= 256) SMO_CASE(false, 1, 256); else if (ws <= 512) SMO_CASE(false, 2, 256); else SMO_CASE(false, 2, 512);
    } else {
        if (ws <= 256) SMO_CASE(true, 1, 256); else if (ws <= 512) SMO_CASE(true, 2, 256); else SMO_CASE(true, 2, 512);
    }
#undef SMO_CASE
    return TSVM_OK;
}

}  // namespace tsvm

using namespace tsvm;

// Bytes a solver may use for its row buffer / kernel-row cache: what tsvm_set_row_cache_bytes or the environment
// variable TSVM_ROW_CACHE_MB asked for, else 45 % of the device's memory (a fixed fraction of the total, not of
// what happens to be free, so that consecutive solvers of the same problem ask for the same block and get it
// back from the library's pool).
static long long g_row_cache_bytes = -1;
static size_t row_cache_budget() {
    if (g_row_cache_bytes >= 0) return (size_t) g_row_cache_bytes;
    if (const char *e = getenv("TSVM_ROW_CACHE_MB")) return (size_t) strtoull(e, nullptr, 10) << 20;
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) { cudaGetLastError(); return (size_t) 8 << 30; }
    return (size_t) ((double) total_b * 0.45);
}

struct tsvm_ws {
    int n_max = 0, ws_max = 0;
    int cand_cap = 0;               // entries per list of cand_f / cand_id
    SelectState *state = nullptr;
    int *hist = nullptr, *ticket = nullptr, *count = nullptr;
    double *cand_f = nullptr;
    int *cand_id = nullptr;
};

extern "C" {

void tsvm_set_row_cache_bytes(long long bytes) { g_row_cache_bytes = bytes; }

tsvm_status tsvm_ws_create(int n_max, int ws_max, tsvm_ws **out) {
    TSVM_REQUIRE(out && n_max > 0 && ws_max > 0 && ws_max <= MERGE_MAX_WANT, "ws_create: bad arguments");
    tsvm_ws *w = new tsvm_ws;
    w->n_max = n_max; w->ws_max = ws_max;
    w->cand_cap = 2 * ws_max;       // room for the whole threshold digit of an early-resolved list
    tsvm_status s = dev_alloc(&w->state, MAX_LISTS);
    if (s == TSVM_OK) s = dev_alloc(&w->hist, MAX_LISTS * RADIX_BINS);
    if (s == TSVM_OK) s = dev_alloc(&w->ticket, 1);
    if (s == TSVM_OK) s = dev_alloc(&w->count, 1);
    if (s == TSVM_OK) s = dev_alloc(&w->cand_f, (size_t) MAX_LISTS * w->cand_cap);
    if (s == TSVM_OK) s = dev_alloc(&w->cand_id, (size_t) MAX_LISTS * w->cand_cap);
    if (s != TSVM_OK) { tsvm_ws_destroy(w); return s; }
    *out = w;
    return TSVM_OK;
}

void tsvm_ws_destroy(tsvm_ws *w) {
    if (!w) return;
    pool_free_many({w->state, w->hist, w->ticket, w->count, w->cand_f, w->cand_id});
    delete w;
}

// The selection in one cooperative launch (select_fused_kernel). Candidate lists of `cap` >= want entries each
// (stride cap): the `want` best of every list are among them; mode says what happens to them on the device.
struct FusedExtra {
    int mode = FUSED_CANDIDATES;
    int *out_ids = nullptr;                       // FUSED_MERGE
    double *sorted_f = nullptr;                   // FUSED_SORT
    int *sorted_id = nullptr;
    int *shift_ids = nullptr;                     // optional rotation of the working set first
    int shift_q = 0;
    unsigned char *shift_flags = nullptr;
    const int *stop = nullptr;
};

static size_t fused_smem_bytes(int lists, int cap, int mode) {
    size_t b = (size_t) lists * RADIX_BINS * sizeof(int);
    int P = 1;
    while (P < cap) P <<= 1;
    if (mode == FUSED_MERGE && merge_smem_bytes(cap) > b) b = merge_smem_bytes(cap);
    if (mode == FUSED_SORT && (size_t) P * 20 + 8 > b) b = (size_t) P * 20 + 8;
    return b;
}

static tsvm_status ws_candidates_cap(tsvm_ws *w, int solver_kind, int n, const double *f_dev, const double *alpha_dev,
                                     const int *y_dev, const unsigned char *in_ws_dev, double Cp, double Cn, int want,
                                     int cap, int id_offset, double *cand_f_dev, int *cand_id_dev, cudaStream_t st,
                                     const FusedExtra &x = FusedExtra()) {
    const int lists = solver_kind == TSVM_SOLVER_C ? 2 : 4;
    static int resident_blocks[MAX_DEVICES] = {0};
    int dev = 0;
    TSVM_CUDA(cudaGetDevice(&dev));
    int &max_blocks = resident_blocks[dev & (MAX_DEVICES - 1)];
    if (!max_blocks) {
        const size_t smem_max = fused_smem_bytes(MAX_LISTS, MERGE_MAX_LEN, FUSED_SORT) > fused_smem_bytes(MAX_LISTS, MERGE_MAX_LEN, FUSED_MERGE)
                                    ? fused_smem_bytes(MAX_LISTS, MERGE_MAX_LEN, FUSED_SORT)
                                    : fused_smem_bytes(MAX_LISTS, MERGE_MAX_LEN, FUSED_MERGE);
        TSVM_CUDA(cudaFuncSetAttribute(select_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_max));
        int sms = 0, coop = 0;
        TSVM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        TSVM_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        TSVM_REQUIRE(coop, "working-set selection needs a device that supports cooperative launches");
        max_blocks = sms;                         // one 1024-thread block per SM: always resident together
    }
    SelectArgs a;
    a.solver_kind = solver_kind; a.n = n; a.f = f_dev; a.alpha = alpha_dev; a.y = y_dev; a.in_ws = in_ws_dev;
    a.Cp = Cp; a.Cn = Cn; a.st = w->state; a.hist = w->hist; a.ticket = w->ticket; a.want = want; a.cap = cap;
    a.id_offset = id_offset; a.cand_f = cand_f_dev; a.cand_id = cand_id_dev; a.mode = x.mode; a.out_ids = x.out_ids;
    a.out_count = w->count; a.sorted_f = x.sorted_f; a.sorted_id = x.sorted_id; a.shift_ids = x.shift_ids;
    a.shift_q = x.shift_q; a.shift_flags = x.shift_flags; a.stop = x.stop;
    int grid = ceil_div(n, FUSED_THREADS * 2);
    if (grid > max_blocks) grid = max_blocks;
    if (grid < (x.mode == FUSED_SORT ? lists : 1)) grid = x.mode == FUSED_SORT ? lists : 1;
    void *args[] = {&a};
    TSVM_CUDA(cudaLaunchCooperativeKernel((const void *) select_fused_kernel, dim3(grid), dim3(FUSED_THREADS), args,
                                          fused_smem_bytes(lists, cap, x.mode), st));
    count_launch();
    return TSVM_OK;
}

tsvm_status tsvm_ws_candidates(tsvm_ws *w, int solver_kind, int n, const double *f_dev, const double *alpha_dev,
                               const int *y_dev, const unsigned char *in_ws_dev, double Cp, double Cn, int want,
                               int id_offset, double *cand_f_dev, int *cand_id_dev, void *stream) {
    TSVM_REQUIRE(w && f_dev && alpha_dev && y_dev && cand_f_dev && cand_id_dev && n > 0 && want > 0 &&
                 want <= w->ws_max && solver_kind >= 0 && solver_kind <= 2, "ws_candidates: bad arguments");
    return ws_candidates_cap(w, solver_kind, n, f_dev, alpha_dev, y_dev, in_ws_dev, Cp, Cn, want, want, id_offset,
                             cand_f_dev, cand_id_dev, (cudaStream_t) stream);
}

static tsvm_status ws_merge_impl(tsvm_ws *w, int solver_kind, const double *cand_f_dev, const int *cand_id_dev, int len,
                                 int seg_len, int want, int *out_ids_dev, cudaStream_t st) {
    const size_t smem = merge_smem_bytes(len);
    TSVM_ONCE_PER_DEVICE(TSVM_CUDA(cudaFuncSetAttribute(select_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        (int) merge_smem_bytes(MERGE_MAX_LEN))));
    TSVM_LAUNCH(select_merge_kernel, 1, MERGE_THREADS, smem, st, solver_kind, cand_f_dev, cand_id_dev, len, want,
                out_ids_dev, w->count, seg_len);
    return TSVM_OK;
}

tsvm_status tsvm_ws_merge(tsvm_ws *w, int solver_kind, const double *cand_f_dev, const int *cand_id_dev, int len,
                          int want, int *out_ids_dev, void *stream) {
    TSVM_REQUIRE(w && cand_f_dev && cand_id_dev && out_ids_dev && len > 0 && len <= MERGE_MAX_LEN && want > 0 &&
                 want <= MERGE_MAX_WANT, "ws_merge: bad arguments (len=%d want=%d)", len, want);
    return ws_merge_impl(w, solver_kind, cand_f_dev, cand_id_dev, len, 0, want, out_ids_dev, (cudaStream_t) stream);
}

static tsvm_status ws_sort_impl(int solver_kind, const double *in_f, const int *in_id, int len, double *out_f, int *out_id,
                                int out_len, cudaStream_t st) {
    int P = 1;
    while (P < len) P <<= 1;
    const size_t smem = (size_t) P * 12 + 8 + (size_t) P * 8;
    TSVM_ONCE_PER_DEVICE(TSVM_CUDA(cudaFuncSetAttribute(select_sort_candidates_kernel,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        (int) ((size_t) MERGE_MAX_LEN * 20 + 8))));
    TSVM_LAUNCH(select_sort_candidates_kernel, solver_kind == TSVM_SOLVER_C ? 2 : 4, MERGE_THREADS, smem, st,
                solver_kind, in_f, in_id, len, out_f, out_id, out_len);
    return TSVM_OK;
}

tsvm_status tsvm_ws_sort_candidates(tsvm_ws *w, int solver_kind, double *cand_f_dev, int *cand_id_dev, int len,
                                    void *stream) {
    TSVM_REQUIRE(w && cand_f_dev && cand_id_dev && len > 0 && len <= MERGE_MAX_LEN && solver_kind >= 0 &&
                 solver_kind <= 2, "ws_sort_candidates: bad arguments (len=%d)", len);
    return ws_sort_impl(solver_kind, cand_f_dev, cand_id_dev, len, cand_f_dev, cand_id_dev, len, (cudaStream_t) stream);
}

tsvm_status tsvm_ws_merge_sorted(tsvm_ws *w, int solver_kind, const double *cand_f_dev, const int *cand_id_dev, int len,
                                 int seg_len, int want, int *out_ids_dev, void *stream) {
    TSVM_REQUIRE(w && cand_f_dev && cand_id_dev && out_ids_dev && len > 0 && len <= MERGE_MAX_LEN && want > 0 &&
                 want <= MERGE_MAX_WANT && seg_len > 0 && len % seg_len == 0 && len / seg_len <= MERGE_THREADS,
                 "ws_merge_sorted: bad arguments (len=%d seg_len=%d want=%d)", len, seg_len, want);
    return ws_merge_impl(w, solver_kind, cand_f_dev, cand_id_dev, len, seg_len, want, out_ids_dev, (cudaStream_t) stream);
}

tsvm_status tsvm_select_working_set(tsvm_ws *w, int solver_kind, int n, const double *f_dev, const double *alpha_dev,
                                    const int *y_dev, const unsigned char *in_ws_dev, double Cp, double Cn, int want,
                                    int *out_ids_dev, void *stream) {
    TSVM_REQUIRE(w && f_dev && alpha_dev && y_dev && out_ids_dev && n > 0 && want > 0 && want <= w->ws_max &&
                 solver_kind >= 0 && solver_kind <= 2, "select_working_set: bad arguments");
    const int cap = 2 * want <= w->cand_cap ? 2 * want : (want <= w->cand_cap ? w->cand_cap : want);
    TSVM_REQUIRE(cap >= want, "select_working_set: candidate buffers hold %d entries, %d wanted", w->cand_cap, want);
    FusedExtra x;
    x.mode = FUSED_MERGE;
    x.out_ids = out_ids_dev;
    return ws_candidates_cap(w, solver_kind, n, f_dev, alpha_dev, y_dev, in_ws_dev, Cp, Cn, want, cap, 0, w->cand_f,
                             w->cand_id, (cudaStream_t) stream, x);
}

// ---- working-set selection without any allocation --------------------------------------------------
// Scratch of tsvm_select_working_set_static: the per-list selection state, the radix histograms, the
// ticket / count words and the candidate lists for up to TSVM_STATIC_WS_MAX wanted ids and four
// lists. It is a fixed part of the library image: every GPU that loads the library holds these
// bytes until the process exits.
constexpr int STATIC_WS_MAX = TSVM_STATIC_WS_MAX;
constexpr size_t STATIC_OFF_STATE = 0;                                                   // SelectState[4]
constexpr size_t STATIC_OFF_HIST = 256;                                                  // int[4 * 4096]
constexpr size_t STATIC_OFF_TICKET = STATIC_OFF_HIST + sizeof(int) * MAX_LISTS * RADIX_BINS;   // int
constexpr size_t STATIC_OFF_COUNT = STATIC_OFF_TICKET + 128;                             // int
constexpr size_t STATIC_OFF_CAND_F = STATIC_OFF_COUNT + 128;                             // double[4 * 1024]
constexpr size_t STATIC_OFF_CAND_ID = STATIC_OFF_CAND_F + sizeof(double) * MAX_LISTS * STATIC_WS_MAX;
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_OFF_CAND_ID + sizeof(int) * MAX_LISTS * STATIC_WS_MAX;
static_assert(sizeof(SelectState) * MAX_LISTS <= STATIC_OFF_HIST, "selection state does not fit its slot");
static __device__ __align__(256) unsigned char g_static_select_scratch[STATIC_SCRATCH_BYTES];

// In host code the array's name is only a stand-in for the symbol, not a device address: the address
// is asked from the runtime once per device (with that device current) and remembered. The cache is
// written without a lock by whichever host thread calls first on a device; every writer stores the same
// value, so concurrent first calls are harmless.
constexpr int STATIC_MAX_DEVICES = MAX_DEVICES;
static unsigned char *g_static_scratch_addr[STATIC_MAX_DEVICES] = {nullptr};

tsvm_status tsvm_select_working_set_static(int solver_kind, int n, const double *f_dev, const double *alpha_dev,
                                           const int *y_dev, const unsigned char *in_ws_dev, double Cp, double Cn,
                                           int want, int *out_ids_dev, void *stream) {
    TSVM_REQUIRE(f_dev && alpha_dev && y_dev && out_ids_dev && n > 0 && want > 0 && solver_kind >= 0 &&
                 solver_kind <= 2, "select_working_set_static: bad arguments");
    TSVM_REQUIRE(want <= STATIC_WS_MAX,
                 "select_working_set_static: %d ids wanted, the built-in scratch holds at most %d "
                 "(use tsvm_select_working_set with a tsvm_ws for more)", want, STATIC_WS_MAX);
    int dev = 0;
    TSVM_CUDA(cudaGetDevice(&dev));
    TSVM_REQUIRE(dev >= 0 && dev < STATIC_MAX_DEVICES, "select_working_set_static: device ordinal %d not supported", dev);
    if (!g_static_scratch_addr[dev]) {
        void *p = nullptr;
        TSVM_CUDA(cudaGetSymbolAddress(&p, g_static_select_scratch));
        g_static_scratch_addr[dev] = static_cast<unsigned char *>(p);
    }
    unsigned char *base = g_static_scratch_addr[dev];
    tsvm_ws view;                      // a view over the static array; owns nothing, frees nothing
    view.n_max = n;
    view.ws_max = STATIC_WS_MAX;
    view.cand_cap = STATIC_WS_MAX;
    view.state = reinterpret_cast<SelectState *>(base + STATIC_OFF_STATE);
    view.hist = reinterpret_cast<int *>(base + STATIC_OFF_HIST);
    view.ticket = reinterpret_cast<int *>(base + STATIC_OFF_TICKET);
    view.count = reinterpret_cast<int *>(base + STATIC_OFF_COUNT);
    view.cand_f = reinterpret_cast<double *>(base + STATIC_OFF_CAND_F);
    view.cand_id = reinterpret_cast<int *>(base + STATIC_OFF_CAND_ID);
    // the selection kernel's first phase zeroes the state, the histograms and the ticket and resets the
    // candidate ids on every call, so nothing of an earlier call's contents is read.
    return tsvm_select_working_set(&view, solver_kind, n, f_dev, alpha_dev, y_dev, in_ws_dev, Cp, Cn, want,
                                   out_ids_dev, stream);
}

tsvm_status tsvm_local_smo(int solver_kind, int ws_size, const float *kww_dev, const float *diag_ws_dev,
                           const int *y_ws_dev, const double *f_ws_dev, double *alpha_ws_dev, double *alpha_diff_dev,
                           double Cp, double Cn, double eps, int max_iter, double *diff_dev, void *stream) {
    TSVM_REQUIRE(ws_size > 0 && ws_size <= 1024 && kww_dev && diag_ws_dev && y_ws_dev && f_ws_dev && alpha_ws_dev &&
                 alpha_diff_dev && diff_dev, "local_smo: bad arguments (ws=%d)", ws_size);
    return launch_local_smo(solver_kind, ws_size, kww_dev, diag_ws_dev, y_ws_dev, f_ws_dev, alpha_ws_dev,
                            alpha_diff_dev, Cp, Cn, eps, max_iter, diff_dev, nullptr, nullptr, (cudaStream_t) stream);
}

tsvm_status tsvm_rho_partials(int n, const double *f_dev, const double *alpha_dev, const int *y_dev, double Cp,
                              double Cn, double *out13_dev, void *stream) {
    TSVM_REQUIRE(n > 0 && f_dev && alpha_dev && y_dev && out13_dev, "rho_partials: bad arguments");
    TSVM_LAUNCH(rho_obj_kernel, 1, 1024, 0, (cudaStream_t) stream, n, f_dev, alpha_dev, y_dev, Cp, Cn, out13_dev);
    return TSVM_OK;
}

tsvm_status tsvm_update_f(double *f_dev, int n, const double *alpha_diff_dev, int ws_size, const float *rows_dev,
                          long long ld, void *stream) {
    TSVM_REQUIRE(f_dev && alpha_diff_dev && rows_dev && n > 0 && ws_size > 0 && ws_size <= 1024 && ld >= n,
                 "update_f: bad arguments (at most 1024 rows per call)");
    TSVM_LAUNCH(update_f_kernel, update_f_grid(n), 128, 0, (cudaStream_t) stream, f_dev, n, alpha_diff_dev, ws_size,
                0, 0, rows_dev, ld, rows_vec_ok(rows_dev, ld), 0, ws_size, update_f_cols(n), (const int *) nullptr);
    return TSVM_OK;
}

int tsvm_working_set_size(int n_instances, int n_features, size_t max_mem_bytes, size_t used_bytes) {
    if (max_mem_bytes < used_bytes) return -1;
    // max2power(x) = 2^floor(log2f(x)) (include/thundersvm/util/common.h:20-23)
    auto max2power = [](double x) -> long long { return (long long) exp2(floor(log2f((float) x))); };
    const size_t free_mem = max_mem_bytes - used_bytes;
    long long a = max2power((double) n_instances);
    long long b = max2power((double) (free_mem / sizeof(float) / ((size_t) n_instances + n_features)));
    if (b > 1024) b = 1024;
    return (int) (a < b ? a : b);
}

}  // extern "C"

// Solver state that persists across outer iterations.
// How many iterations are queued between two reads of the device's verdict. The queue hides the host's wake-up
// and launch latency behind the device's work; the price is at most that many no-op iterations after the one
// that ends the solve.
enum { MAX_QUEUED = 32 };
static int sync_every() {
    static const int k = [] {
        const char *e = getenv("TSVM_SYNC_EVERY");
        const int v = e ? atoi(e) : 8;
        return v < 1 ? 1 : (v > MAX_QUEUED ? (int) MAX_QUEUED : v);
    }();
    return k;
}

struct tsvm_solver {
    // Events of one queued iteration: phase boundaries on the first stream, start and end of the local solver
    struct IterEvents {
        cudaEvent_t ph[5] = {nullptr, nullptr, nullptr, nullptr, nullptr}, l0 = nullptr, l1 = nullptr;
    };

    tsvm_km *km = nullptr;
    int kind = 0, ws = 0, q = 0, n = 0;
    const int *y = nullptr;
    double *alpha = nullptr, *f = nullptr;
    double eps = 0, Cp = 0, Cn = 0;
    long long ld = 0;
    cudaStream_t st = nullptr;
    // device buffers
    int *ids = nullptr, *y_ws = nullptr;
    float *rows = nullptr, *kww = nullptr, *diag_ws = nullptr;
    double *f_ws = nullptr, *a_ws = nullptr, *alpha_diff = nullptr, *diff = nullptr, *red = nullptr;
    unsigned char *in_ws = nullptr;
    tsvm_ws *sel = nullptr;
    double *diff_host = nullptr;
    // end-of-iteration state on the device, its pinned copy, and the events of the queued iterations
    SolverCtl *ctl = nullptr, *ctl_host = nullptr;
    IterEvents evs[MAX_QUEUED];
    int max_iter = -1;              // iteration cap applied on the device; -1: none
    bool stopped = false;           // the device stopped the queue (done, capped or an error)
    // overlapped iteration: second stream, fork / join events, operand planes of the working set
    bool overlap = true;
    cudaStream_t st2 = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_fork2 = nullptr, ev_join = nullptr;
    float *ws_hi = nullptr, *ws_lo = nullptr, *ws_sd = nullptr, *ws_unscale = nullptr;
    // kernel-row cache (cache_assign_kernel): the row buffer holds cache_cap rows; directory and per-iteration lists
    long long cache_cap = 0;
    int *slot_of = nullptr, *inst_of = nullptr, *stamp = nullptr, *row_slot = nullptr, *miss_ids = nullptr,
        *miss_slot = nullptr, *victims = nullptr;
    long long *cache_ctr = nullptr;
    float *miss_hi = nullptr, *miss_lo = nullptr, *miss_sd = nullptr, *miss_unscale = nullptr;
    long long hits = 0, misses = 0, row_blocks = 0, row_blocks_saved = 0;
    // iteration state (csmosolver.cpp:51-57)
    long long iter = 0, local_iter = 0, rows_made = 0, launches0 = 0;
    int local_max_iter = 0;
    double diff0 = 0;
    double t_sel = 0, t_rows = 0, t_loc = 0, t_upd = 0;
    bool done = false;
    std::chrono::steady_clock::time_point t_begin;

    ~tsvm_solver() {
        pool_free_many({ids, y_ws, rows, kww, diag_ws, f_ws, a_ws, alpha_diff, diff, red, in_ws, ws_hi, ws_lo, ws_sd,
                        ws_unscale, slot_of, inst_of, stamp, row_slot, miss_ids, miss_slot, victims, cache_ctr, miss_hi,
                        miss_lo, miss_sd, miss_unscale, ctl});
        tsvm_ws_destroy(sel);
        if (diff_host) pinned_free(diff_host);
        if (ctl_host) pinned_free(ctl_host);
        for (auto &E : evs) {
            for (auto e : E.ph) if (e) cudaEventDestroy(e);
            for (auto e : {E.l0, E.l1}) if (e) cudaEventDestroy(e);
        }
        for (auto e : {ev_fork, ev_fork2, ev_join}) if (e) cudaEventDestroy(e);
        if (st2) cudaStreamDestroy(st2);
    }

    tsvm_status ensure_ws_planes() {
        if (ws_hi) return TSVM_OK;
        const size_t words = (km_plane_row_bytes(km) * (size_t) ws + 3) / 4;
        TSVM_TRY(dev_alloc(&ws_hi, words));
        TSVM_TRY(dev_alloc(&ws_lo, words));
        TSVM_TRY(dev_alloc(&ws_sd, (size_t) ws));
        TSVM_TRY(dev_alloc(&ws_unscale, (size_t) ws));
        return TSVM_OK;
    }

    tsvm_status ensure_miss_planes() {
        if (miss_hi) return TSVM_OK;
        const size_t words = (km_plane_row_bytes(km) * (size_t) ws + 3) / 4;
        TSVM_TRY(dev_alloc(&miss_hi, words));
        TSVM_TRY(dev_alloc(&miss_lo, words));
        TSVM_TRY(dev_alloc(&miss_sd, (size_t) ws));
        TSVM_TRY(dev_alloc(&miss_unscale, (size_t) ws));
        return TSVM_OK;
    }

    // Row buffer = kernel-row cache: as many rows as the budget allows (tsvm_set_row_cache_bytes), at least the
    // working set plus one batch of new rows, at most one row per instance. A failed allocation halves the request.
    tsvm_status alloc_rows() {
        const long long floor_rows = (long long) ws + q;
        long long want = (long long) (row_cache_budget() / (sizeof(float) * (size_t) ld));
        if (want > n) want = n;
        if (want < floor_rows) want = floor_rows;
        for (;;) {
            const tsvm_status s = dev_alloc(&rows, (size_t) want * ld);
            if (s == TSVM_OK) break;
            if (s != TSVM_ERR_OOM || want == floor_rows) return s;
            want = want / 2 > floor_rows ? want / 2 : floor_rows;
        }
        cache_cap = want;
        TSVM_TRY(dev_alloc(&slot_of, (size_t) n));
        TSVM_TRY(dev_alloc(&inst_of, (size_t) cache_cap));
        TSVM_TRY(dev_alloc(&stamp, (size_t) cache_cap));
        TSVM_TRY(dev_alloc(&row_slot, (size_t) ws));
        TSVM_TRY(dev_alloc(&miss_ids, (size_t) ws));
        TSVM_TRY(dev_alloc(&miss_slot, (size_t) ws));
        TSVM_TRY(dev_alloc(&victims, (size_t) ws));
        TSVM_TRY(dev_alloc(&cache_ctr, (size_t) CACHE_CTRS));
        TSVM_LAUNCH(fill_int_kernel, 296, 256, 0, st, slot_of, (long long) n, -1);
        TSVM_LAUNCH(fill_int_kernel, 296, 256, 0, st, inst_of, cache_cap, -1);
        TSVM_CUDA(cudaMemsetAsync(stamp, 0, sizeof(int) * (size_t) cache_cap, st));
        TSVM_CUDA(cudaMemsetAsync(row_slot, 0, sizeof(int) * (size_t) ws, st));
        TSVM_CUDA(cudaMemsetAsync(cache_ctr, 0, sizeof(long long) * CACHE_CTRS, st));
        return TSVM_OK;
    }

    tsvm_status init() {
        TSVM_TRY(dev_alloc(&ids, (size_t) ws));
        TSVM_TRY(dev_alloc(&y_ws, (size_t) ws));
        TSVM_TRY(alloc_rows());
        TSVM_TRY(dev_alloc(&kww, (size_t) ws * ws));
        TSVM_TRY(dev_alloc(&diag_ws, (size_t) ws));
        TSVM_TRY(dev_alloc(&f_ws, (size_t) ws));
        TSVM_TRY(dev_alloc(&a_ws, (size_t) ws));
        TSVM_TRY(dev_alloc(&alpha_diff, (size_t) ws));
        TSVM_TRY(dev_alloc(&diff, 4));
        TSVM_TRY(dev_alloc(&red, 16));   // >= RHO_VALS
        TSVM_TRY(dev_alloc(&in_ws, (size_t) n));
        TSVM_CUDA(cudaMemsetAsync(in_ws, 0, (size_t) n, st));
        TSVM_TRY(tsvm_ws_create(n, ws, &sel));
        TSVM_TRY(pinned_alloc((void **) &diff_host, 16 * sizeof(double)));
        TSVM_TRY(dev_alloc(&ctl, 1));
        TSVM_TRY(pinned_alloc((void **) &ctl_host, sizeof(SolverCtl)));
        memset(ctl_host, 0, sizeof(SolverCtl));
        ctl_host->prev = ctl_host->last = ctl_host->second_last = INFINITY;     // csmosolver.cpp:51-57
        TSVM_CUDA(cudaMemcpyAsync(ctl, ctl_host, sizeof(SolverCtl), cudaMemcpyHostToDevice, st));
        TSVM_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
        TSVM_CUDA(cudaEventCreateWithFlags(&ev_fork2, cudaEventDisableTiming));
        TSVM_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
        {
            int lo_prio = 0, hi_prio = 0;
            TSVM_CUDA(cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
            TSVM_CUDA(cudaStreamCreateWithPriority(&st2, cudaStreamNonBlocking, hi_prio));
        }
        // local iteration cap: max(100000, 100 * ws) (csmosolver.cpp:49)
        local_max_iter = ws > INT_MAX / 100 ? INT_MAX : (100 * ws > 100000 ? 100 * ws : 100000);
        return init_f();
    }

    // init_f (csmosolver.cpp:189-214): f -= sum over the initially non-zero alphas
    tsvm_status init_f() {
        std::vector<double> a_h(n);
        std::vector<int> y_h(n);
        TSVM_CUDA(cudaMemcpyAsync(a_h.data(), alpha, sizeof(double) * n, cudaMemcpyDeviceToHost, st));
        TSVM_CUDA(cudaMemcpyAsync(y_h.data(), y, sizeof(int) * n, cudaMemcpyDeviceToHost, st));
        TSVM_CUDA(cudaStreamSynchronize(st));
        std::vector<int> bi;
        std::vector<double> bd;
        auto flush = [&]() -> tsvm_status {
            if (bi.empty()) return TSVM_OK;
            const int m = (int) bi.size();
            TSVM_CUDA(cudaMemcpyAsync(ids, bi.data(), sizeof(int) * m, cudaMemcpyHostToDevice, st));
            TSVM_CUDA(cudaMemcpyAsync(alpha_diff, bd.data(), sizeof(double) * m, cudaMemcpyHostToDevice, st));
            TSVM_TRY(tsvm_km_rows_by_index(km, ids, m, rows, ld, st));
            TSVM_LAUNCH(update_f_kernel, update_f_grid(n), 128, 0, st, f, n, alpha_diff, m, 0, 0, rows, ld,
                        rows_vec_ok(rows, ld), 0, m, update_f_cols(n), (const int *) nullptr);
            TSVM_CUDA(cudaStreamSynchronize(st));
            rows_made += m;
            bi.clear(); bd.clear();
            return TSVM_OK;
        };
        for (int i = 0; i < n; ++i) {
            if (a_h[i] != 0) { bi.push_back(i); bd.push_back(-a_h[i] * y_h[i]); }
            if ((int) bi.size() == ws) TSVM_TRY(flush());
        }
        return flush();
    }

    // Queues one outer iteration of csmosolver.cpp:59-120, number `it`, without waiting for it. Its last launch
    // applies the reference's termination rules (csmosolver.cpp:86-111) on the device; every launch of an
    // iteration queued after the one that ended the solve is a no-op.
    //
    // Overlapped form (dense data on the CTA-pair tensor engine, every iteration but the first): the local
    // solver only needs the ws x ws block of kernel values, not the q full rows. The block's q new rows are
    // computed first by a small launch of the same engine against the working set's own operand planes
    // (bit-identical to the values the full rows will hold: same planes, same slab order), its old rows are
    // gathered from the rows already in the buffer, and the one-CTA local solver then runs on a second stream
    // while the q x n launch - which leaves one SM pair free for it - fills the row buffer. Both meet before
    // the f update.
    tsvm_status enqueue_iteration(long long it, const IterEvents &E) {
        const int t0 = it == 0 ? 0 : q, n_new = it == 0 ? ws : q;          // iteration 0 fills the whole working set
        const bool overlapped = overlap && it > 0 && st2 && km_pair_engine(km, st);
        const int row_block = km_pair_engine(km, st) ? 256 : 64;           // requested rows per tile of the engine
        const int *n_miss_dev = reinterpret_cast<const int *>(cache_ctr);
        const int *stop = &ctl->stop;
        TSVM_CUDA(cudaEventRecord(E.ph[0], st));
        if (it == 0) {
            TSVM_TRY(tsvm_select_working_set(sel, kind, n, f, alpha, y, nullptr, Cp, Cn, ws, ids, st));
        } else {
            // rotation of the working set (old second half -> first half, flags) and the selection of the new
            // second half: one cooperative launch
            FusedExtra x;
            x.mode = FUSED_MERGE;
            x.out_ids = ids + q;
            x.shift_ids = ids; x.shift_q = q; x.shift_flags = in_ws;
            x.stop = stop;
            TSVM_TRY(ws_candidates_cap(sel, kind, n, f, alpha, y, in_ws, Cp, Cn, q, 2 * q <= sel->cand_cap ? 2 * q : q, 0,
                                       sel->cand_f, sel->cand_id, st, x));
        }
        if (overlapped) {
            // The block's new rows need the members' planes and nothing else: the second stream starts on them
            // (new members against all members, from the members' own operand planes) while the first one still
            // runs the cache directory, i.e. before the big launch takes all SM pairs but one.
            TSVM_TRY(ensure_ws_planes());
            TSVM_TRY(ensure_miss_planes());
            TSVM_TRY(km_gather_planes(km, ids, ws, nullptr, ws_hi, ws_lo, ws_sd, ws_unscale, st));
            TSVM_CUDA(cudaEventRecord(ev_fork, st));
            TSVM_CUDA(cudaStreamWaitEvent(st2, ev_fork, 0));
            const size_t rb = km_plane_row_bytes(km);
            const InstancePlanes members{ws_hi, ws_lo, ws_sd, ws_unscale, ws};
            const RowPlanes new_members{reinterpret_cast<const float *>(reinterpret_cast<const char *>(ws_hi) + (size_t) q * rb),
                                        reinterpret_cast<const float *>(reinterpret_cast<const char *>(ws_lo) + (size_t) q * rb),
                                        ws_sd + q, ws_unscale + q};
            TSVM_TRY(km_rows_planes_on(km, members, new_members, q, kww + (size_t) q * ws, ws, st2));
        }
        // cache directory: hits point at their rows, misses get the least recently used rows
        TSVM_LAUNCH(cache_assign_kernel, 1, CACHE_THREADS, 0, st, ids, t0, n_new, (int) (it + 1), slot_of, inst_of, stamp,
                    (int) cache_cap, row_slot, miss_ids, miss_slot, victims, cache_ctr, row_block, stop);
        TSVM_CUDA(cudaEventRecord(E.ph[1], st));
        if (!overlapped) {
            // the engine computes the missing rows only (their number is read on the device) into their cache rows
            km->rows_m_dev = n_miss_dev; km->rows_slot_dev = miss_slot;
            const tsvm_status rs = tsvm_km_rows_by_index(km, miss_ids, n_new, rows, ld, st);
            km->rows_m_dev = nullptr; km->rows_slot_dev = nullptr;
            TSVM_TRY(rs);
        } else {
            TSVM_TRY(km_gather_planes(km, miss_ids, q, n_miss_dev, miss_hi, miss_lo, miss_sd, miss_unscale, st));
            TSVM_CUDA(cudaEventRecord(ev_fork2, st));
            // second stream, after the directory: block rows 0..q-1 and the slot vectors by gather from the rows in
            // the buffer, then the local solver
            TSVM_CUDA(cudaStreamWaitEvent(st2, ev_fork2, 0));
            TSVM_LAUNCH(gather_ws_kernel, ws, 256, 0, st2, ws, q, 0, ids, rows, ld, km->diag, y, f, alpha, kww, diag_ws,
                        y_ws, f_ws, a_ws, q, row_slot);
            TSVM_CUDA(cudaEventRecord(E.l0, st2));
            TSVM_TRY(launch_local_smo(kind, ws, kww, diag_ws, y_ws, f_ws, a_ws, alpha_diff, Cp, Cn, eps, local_max_iter,
                                      diff, ids, alpha, st2, stop));
            TSVM_CUDA(cudaEventRecord(E.l1, st2));
            // the rows that were in the buffer already can be applied to f at once (HBM-bound, next to the
            // tensor-bound launch); the new rows follow on the first stream
            TSVM_LAUNCH(update_f_kernel, update_f_grid(n), 128, 0, st2, f, n, alpha_diff, ws, q, 0, rows, ld,
                        rows_vec_ok(rows, ld), 0, q, update_f_cols(n), row_slot);
            TSVM_CUDA(cudaEventRecord(ev_join, st2));
            // first stream: the missing rows against all instances, on all SM pairs but one
            const InstancePlanes all{km->Xhi, km->Xlo, km->self_dot, km->x_unscale, km->n};
            const RowPlanes miss_rows{miss_hi, miss_lo, miss_sd, miss_unscale};
            km->reserve_clusters = 1;
            km->rows_m_dev = n_miss_dev; km->rows_slot_dev = miss_slot;
            const tsvm_status rs = km_rows_planes_on(km, all, miss_rows, q, rows, ld, st);
            km->reserve_clusters = 0;
            km->rows_m_dev = nullptr; km->rows_slot_dev = nullptr;
            TSVM_TRY(rs);
        }
        TSVM_CUDA(cudaEventRecord(E.ph[2], st));
        if (!overlapped) {
            TSVM_LAUNCH(gather_ws_kernel, ws, 256, 0, st, ws, q, 0, ids, rows, ld, km->diag, y, f, alpha, kww, diag_ws,
                        y_ws, f_ws, a_ws, ws, row_slot);
            TSVM_CUDA(cudaEventRecord(E.l0, st));
            TSVM_TRY(launch_local_smo(kind, ws, kww, diag_ws, y_ws, f_ws, a_ws, alpha_diff, Cp, Cn, eps, local_max_iter,
                                      diff, ids, alpha, st, stop));
            TSVM_CUDA(cudaEventRecord(E.l1, st));
        } else {
            TSVM_CUDA(cudaStreamWaitEvent(st, ev_join, 0));
        }
        TSVM_CUDA(cudaEventRecord(E.ph[3], st));
        // f -= sum over the old half's rows, then f -= sum over the new half's rows: two launches in every
        // form of the iteration, so that all of them round alike (the first iteration has new rows only)
        if (it == 0) {
            TSVM_LAUNCH(update_f_kernel, update_f_grid(n), 128, 0, st, f, n, alpha_diff, ws, q, 0, rows, ld,
                        rows_vec_ok(rows, ld), 0, ws, update_f_cols(n), row_slot);
        } else {
            if (!overlapped)
                TSVM_LAUNCH(update_f_kernel, update_f_grid(n), 128, 0, st, f, n, alpha_diff, ws, q, 0, rows, ld,
                            rows_vec_ok(rows, ld), 0, q, update_f_cols(n), row_slot);
            TSVM_LAUNCH(update_f_kernel, update_f_grid(n), 128, 0, st, f, n, alpha_diff, ws, q, 0, rows, ld,
                        rows_vec_ok(rows, ld), q, ws, update_f_cols(n), row_slot);
        }
        TSVM_CUDA(cudaEventRecord(E.ph[4], st));
        TSVM_LAUNCH(solver_status_kernel, 1, 32, 0, st, ctl, diff, sel->count, n_new, eps, max_iter, cache_ctr,
                    km->status_dev);
        return TSVM_OK;
    }


    // Queues up to `count` outer iterations, waits once and takes over what the device decided. Fewer than
    // `count` may have run: the termination rules, the iteration cap or an error stop the queue on the device.
    tsvm_status run_iterations(int count) {
        if (count > sync_every()) count = sync_every();
        if (iter == 0) count = 1;                   // the first iteration is read back on its own
        for (int j = 0; j < count; ++j) {
            IterEvents &E = evs[j];
            if (!E.l0) {
                for (auto &e : E.ph) TSVM_CUDA(cudaEventCreate(&e));
                TSVM_CUDA(cudaEventCreate(&E.l0));
                TSVM_CUDA(cudaEventCreate(&E.l1));
            }
            TSVM_TRY(enqueue_iteration(iter + j, E));
        }
        TSVM_CUDA(cudaMemcpyAsync(ctl_host, ctl, sizeof(SolverCtl), cudaMemcpyDeviceToHost, st));
        TSVM_CUDA(cudaStreamSynchronize(st));
        const SolverCtl &c = *ctl_host;
        if (c.engine_status != 0) {
            set_error("dense kernel-row engine reported status %d (a bounded wait ran out)", c.engine_status);
            return TSVM_ERR_DEVICE;
        }
        const int ran = (int) (c.iter - iter);
        for (int j = 0; j < ran; ++j) {
            const IterEvents &E = evs[j];
            float ms;
            cudaEventElapsedTime(&ms, E.ph[0], E.ph[1]); t_sel += ms;
            cudaEventElapsedTime(&ms, E.ph[1], E.ph[2]); t_rows += ms;
            cudaEventElapsedTime(&ms, E.l0, E.l1); t_loc += ms;      // overlapped with the rows phase when both streams run
            cudaEventElapsedTime(&ms, E.ph[3], E.ph[4]); t_upd += ms;
            rows_made += iter + j == 0 ? ws : q;
        }
        hits = c.ctr[CACHE_HITS]; misses = c.ctr[CACHE_MISSES];
        row_blocks = c.ctr[CACHE_BLOCKS]; row_blocks_saved = c.ctr[CACHE_BLOCKS_SAVED];
        iter = c.iter;
        local_iter = c.local_iter;
        diff0 = c.diff0;
        done = c.done != 0;
        stopped = c.stop != 0;
        if (c.short_wanted > 0) {
            // the reference's selection loop never ends here (csmosolver.cpp:131-164); the empty slots were inert
            set_error("working-set selection found %d eligible instances for %d slots (is a class weight or C zero?)",
                      c.short_got, c.short_wanted);
            return TSVM_ERR_INVALID;
        }
        return TSVM_OK;
    }

    tsvm_status outer_iteration() { return run_iterations(1); }

    void fill_stats(tsvm_solve_stats *out, double obj) const {
        out->outer_iters = iter;
        out->local_iters = local_iter;
        out->final_diff = diff0;
        out->objective = obj;
        out->seconds_select = t_sel * 1e-3;
        out->seconds_rows = t_rows * 1e-3;
        out->seconds_local = t_loc * 1e-3;
        out->seconds_update = t_upd * 1e-3;
        out->seconds_total = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_begin).count();
        out->kernel_rows = rows_made;
        out->gpu_launches = launch_count() - launches0;
        out->cache_hits = hits;
        out->cache_misses = misses;
        out->cache_rows = cache_cap;
        out->row_blocks = row_blocks;
        out->row_blocks_saved = row_blocks_saved;
    }

    // rho and objective (csmosolver.cpp:167-187,227-239; nusmosolver.cpp:9-46,120-126)
    tsvm_status finish(double *rho_host, tsvm_solve_stats *stats_host) {
        TSVM_LAUNCH(rho_obj_kernel, 1, 1024, 0, st, n, f, alpha, y, Cp, Cn, red);
        TSVM_CUDA(cudaMemcpyAsync(diff_host, red, RHO_VALS * sizeof(double), cudaMemcpyDeviceToHost, st));
        TSVM_CUDA(cudaStreamSynchronize(st));
        const double *R = diff_host;
        const double obj = -R[4];
        double rho;
        if (kind == TSVM_SOLVER_C) {
            const double nfree = R[0] + R[2];
            rho = nfree != 0 ? (R[1] + R[3]) / nfree : -(fmin(R[5], R[7]) + fmax(R[6], R[8])) / 2;
        } else {
            // nusmosolver.cpp:9-46 works with -f: r = -(min_{I_up}(-f) + max_{I_low}(-f)) / 2
            //                                       =  (max_{I_up} f + min_{I_low} f) / 2
            const double r1 = R[0] != 0 ? R[1] / R[0] : (R[9] + R[10]) / 2;
            const double r2 = R[2] != 0 ? -R[3] / R[2] : (R[11] + R[12]) / 2;
            rho = (r1 - r2) / 2;
            if (kind == TSVM_SOLVER_NU_SVC) {
                const double r = (r1 + r2) / 2;
                TSVM_LAUNCH(scale_kernel, ceil_div(n, 256), 256, 0, st, alpha, n, r);
                TSVM_CUDA(cudaStreamSynchronize(st));
                rho /= r;
            }
        }
        *rho_host = rho;
        if (stats_host) fill_stats(stats_host, obj);
        return TSVM_OK;
    }
};

extern "C" {

// ---- the solver as an object: create / iterate / finish -------------------------------------------
tsvm_status tsvm_solver_create(tsvm_km *km, int solver_kind, const int *y_dev, double *alpha_dev, double *f_dev,
                               double eps, double Cp, double Cn, int ws_size, void *stream, tsvm_solver **out) {
    TSVM_REQUIRE(out && km && y_dev && alpha_dev && f_dev, "solver_create: null argument");
    TSVM_REQUIRE(solver_kind >= 0 && solver_kind <= 2, "solver_create: unknown solver %d", solver_kind);
    const int n = km->n;
    TSVM_REQUIRE(ws_size >= 2 && ws_size <= 1024 && ws_size <= n && (ws_size & (ws_size - 1)) == 0,
                 "solver_create: working-set size %d must be a power of two in [2, min(n, 1024)]", ws_size);
    *out = nullptr;
    tsvm_solver *S = new tsvm_solver;
    S->km = km; S->kind = solver_kind; S->y = y_dev; S->alpha = alpha_dev; S->f = f_dev;
    S->eps = eps; S->Cp = Cp; S->Cn = Cn; S->ws = ws_size; S->q = ws_size / 2; S->n = n;
    S->ld = ((long long) n + 3) & ~3ll;
    S->st = (cudaStream_t) stream;
    S->launches0 = launch_count();
    S->t_begin = std::chrono::steady_clock::now();
    tsvm_status s = S->init();
    if (s != TSVM_OK) { delete S; return s; }
    *out = S;
    return TSVM_OK;
}

tsvm_status tsvm_solver_iterate(tsvm_solver *S, int n_iters, int *done_host) {
    TSVM_REQUIRE(S && n_iters > 0, "solver_iterate: bad arguments");
    for (long long end = S->iter + n_iters; S->iter < end && !S->done;) TSVM_TRY(S->run_iterations((int) (end - S->iter)));
    if (done_host) *done_host = S->done ? 1 : 0;
    return TSVM_OK;
}

tsvm_status tsvm_solver_finish(tsvm_solver *S, double *rho_host, tsvm_solve_stats *stats_host) {
    TSVM_REQUIRE(S && rho_host, "solver_finish: null argument");
    return S->finish(rho_host, stats_host);
}

tsvm_status tsvm_solver_get_stats(const tsvm_solver *S, tsvm_solve_stats *stats_host) {
    TSVM_REQUIRE(S && stats_host, "solver_get_stats: null argument");
    S->fill_stats(stats_host, NAN);
    return TSVM_OK;
}

tsvm_status tsvm_solver_set_overlap(tsvm_solver *S, int enable) {
    TSVM_REQUIRE(S, "solver_set_overlap: null argument");
    S->overlap = enable != 0;
    return TSVM_OK;
}

void tsvm_solver_destroy(tsvm_solver *S) { delete S; }

tsvm_status tsvm_smo_solve(tsvm_km *km, int solver_kind, const int *y_dev, double *alpha_dev, double *f_dev,
                           double eps, double Cp, double Cn, int ws_size, int max_iter, double *rho_host,
                           tsvm_solve_stats *stats_host, void *stream) {
    TSVM_REQUIRE(rho_host, "smo_solve: null argument");
    tsvm_solver *S = nullptr;
    TSVM_TRY(tsvm_solver_create(km, solver_kind, y_dev, alpha_dev, f_dev, eps, Cp, Cn, ws_size, stream, &S));
    tsvm_status s = TSVM_OK;
    // max_iter = k stops after outer iteration k, i.e. k + 1 iterations (csmosolver.cpp:110); applied on the device
    S->max_iter = max_iter;
    while (s == TSVM_OK && !S->stopped) s = S->run_iterations(MAX_QUEUED);
    if (s == TSVM_OK) s = S->finish(rho_host, stats_host);
    delete S;
    return s;
}

}  // extern "C"

// ---- NCCL, bound at run time -------------------------------------------------------------------------
// The library does not link NCCL (a single GPU needs none of it). tsvm_shard_attach_nccl looks the few
// entry points up in the libnccl.so.2 the process already has (or can load) and keeps a communicator.
namespace {
typedef struct ncclComm *ncclComm_t;
struct ncclUniqueIdBytes { char internal[128]; };
enum { NCCL_INT32 = 2, NCCL_FLOAT32 = 7, NCCL_FLOAT64 = 8, NCCL_SUM = 0 };
struct NcclApi {
    int (*GetUniqueId)(ncclUniqueIdBytes *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueIdBytes, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
};
NcclApi &nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return api;
    api.GetUniqueId = (decltype(api.GetUniqueId)) dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank)) dlsym(h, "ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy)) dlsym(h, "ncclCommDestroy");
    api.AllGather = (decltype(api.AllGather)) dlsym(h, "ncclAllGather");
    api.AllReduce = (decltype(api.AllReduce)) dlsym(h, "ncclAllReduce");
    api.GroupStart = (decltype(api.GroupStart)) dlsym(h, "ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd)) dlsym(h, "ncclGroupEnd");
    api.GetErrorString = (decltype(api.GetErrorString)) dlsym(h, "ncclGetErrorString");
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.AllReduce &&
             api.GroupStart && api.GroupEnd && api.GetErrorString;
    return api;
}
}  // namespace
#define TSVM_NCCL(expr)                                                                                  \
    do {                                                                                                 \
        const int r__ = (expr);                                                                          \
        if (r__ != 0) {                                                                                  \
            tsvm::set_error("%s failed: %s", #expr, nccl_api().GetErrorString(r__));                     \
            return TSVM_ERR_CUDA;                                                                        \
        }                                                                                                \
    } while (0)

// Per-rank state of the column-sharded solver. The caller owns the exchange buffers (they are the operands of
// its collectives): cand_f/cand_id [lists * ws], all_f/all_id [world * lists * ws], crow [ws * (dp + 4)] floats,
// cstate [ws * 3] doubles.
struct tsvm_shard {
    tsvm_km *km = nullptr;
    int kind = 0, ws = 0, q = 0, n_local = 0, n_total = 0, lo = 0, hi = 0, world = 1, d = 0, dp = 0;
    const int *y = nullptr;
    double *alpha = nullptr, *f = nullptr;
    double eps = 0, Cp = 0, Cn = 0;
    long long ld = 0;
    cudaStream_t st = nullptr, st2 = nullptr;
    ncclComm_t comm = nullptr;       // set by tsvm_shard_attach_nccl (not owned): the library then runs the exchange steps itself
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_blk = nullptr;
    // timing events of the queued iterations: kernel-row launch (first stream), block + local solver (second)
    struct StepEvents { cudaEvent_t r0 = nullptr, r1 = nullptr, b0 = nullptr, b1 = nullptr; };
    StepEvents evs[MAX_QUEUED];
    int queued = 0;                  // iterations enqueued since the last read of the device's verdict
    SolverCtl *ctl = nullptr, *ctl_host = nullptr;   // termination rules applied on the device (solver_status_kernel)
    double t_rows = 0, t_loc = 0;    // ms
    // exchange buffers (caller's)
    double *cand_f = nullptr, *all_f = nullptr, *cstate = nullptr;
    int *cand_id = nullptr, *all_id = nullptr;
    float *crow = nullptr;
    // own buffers
    int *ids = nullptr, *y_ws = nullptr;
    float *rows = nullptr, *kww = nullptr, *m_hi = nullptr, *m_lo = nullptr, *m_sd = nullptr, *m_unscale = nullptr,
          *m_diag = nullptr;
    double *f_ws = nullptr, *a_ws = nullptr, *alpha_diff = nullptr, *diff = nullptr, *grp_f = nullptr;
    int *grp_id = nullptr;
    unsigned char *in_ws = nullptr;
    tsvm_ws *sel = nullptr;
    size_t row_bytes = 0;
    long long iter = 0, local_iter = 0, rows_made = 0, launches0 = 0;
    int local_max_iter = 0, n_new = 0, slot0 = 0, phase = 0;
    double diff0 = 0;
    bool done = false;
    std::chrono::steady_clock::time_point t_begin;

    ~tsvm_shard() {
        pool_free_many({ids, y_ws, rows, kww, m_hi, m_lo, m_sd, m_unscale, m_diag, f_ws, a_ws, alpha_diff, diff, grp_f,
                        grp_id, in_ws, ctl});
        tsvm_ws_destroy(sel);
        if (ctl_host) pinned_free(ctl_host);
        for (auto e : {ev_fork, ev_join, ev_blk}) if (e) cudaEventDestroy(e);
        for (auto &E : evs)
            for (auto e : {E.r0, E.r1, E.b0, E.b1}) if (e) cudaEventDestroy(e);
        if (st2) cudaStreamDestroy(st2);
    }

    tsvm_status init() {
        TSVM_REQUIRE(km_pair_engine(km, st), "shard solver: needs dense data on the CTA-pair tensor engine "
                                             "(more than 32 features)");
        row_bytes = km_plane_row_bytes(km);
        const size_t plane_words = (row_bytes * (size_t) ws + 3) / 4;
        TSVM_TRY(dev_alloc(&ids, (size_t) ws));
        TSVM_TRY(dev_alloc(&y_ws, (size_t) ws));
        TSVM_TRY(dev_alloc(&rows, (size_t) ws * ld));
        TSVM_TRY(dev_alloc(&kww, (size_t) ws * ws));
        TSVM_TRY(dev_alloc(&m_hi, plane_words));
        TSVM_TRY(dev_alloc(&m_lo, plane_words));
        TSVM_TRY(dev_alloc(&m_sd, (size_t) ws));
        TSVM_TRY(dev_alloc(&m_unscale, (size_t) ws));
        TSVM_TRY(dev_alloc(&m_diag, (size_t) ws));
        TSVM_TRY(dev_alloc(&f_ws, (size_t) ws));
        TSVM_TRY(dev_alloc(&a_ws, (size_t) ws));
        TSVM_TRY(dev_alloc(&alpha_diff, (size_t) ws));
        TSVM_TRY(dev_alloc(&diff, 4));
        TSVM_TRY(dev_alloc(&grp_f, (size_t) world * MAX_LISTS * ws));
        TSVM_TRY(dev_alloc(&grp_id, (size_t) world * MAX_LISTS * ws));
        TSVM_TRY(dev_alloc(&in_ws, (size_t) n_local));
        TSVM_CUDA(cudaMemsetAsync(in_ws, 0, (size_t) n_local, st));
        TSVM_TRY(tsvm_ws_create(n_local, ws, &sel));
        TSVM_TRY(dev_alloc(&ctl, 1));
        TSVM_TRY(pinned_alloc((void **) &ctl_host, sizeof(SolverCtl)));
        memset(ctl_host, 0, sizeof(SolverCtl));
        ctl_host->prev = ctl_host->last = ctl_host->second_last = INFINITY;     // csmosolver.cpp:51-57
        TSVM_CUDA(cudaMemcpyAsync(ctl, ctl_host, sizeof(SolverCtl), cudaMemcpyHostToDevice, st));
        TSVM_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
        TSVM_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
        TSVM_CUDA(cudaEventCreateWithFlags(&ev_blk, cudaEventDisableTiming));
        int lo_prio = 0, hi_prio = 0;
        TSVM_CUDA(cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
        TSVM_CUDA(cudaStreamCreateWithPriority(&st2, cudaStreamNonBlocking, hi_prio));
        local_max_iter = ws > INT_MAX / 100 ? INT_MAX : (100 * ws > 100000 ? 100 * ws : 100000);
        return TSVM_OK;
    }

    // phase A: rotate the working set, then this rank's candidate lists (global ids) into cand_f / cand_id
    tsvm_status candidates(int *lists_out, int *want_out) {
        TSVM_REQUIRE(phase == 0, "shard solver: phases out of order (candidates)");
        const int lists = kind == TSVM_SOLVER_C ? 2 : 4;
        const long long it = iter + queued;         // the iteration being enqueued
        n_new = it == 0 ? ws : q;
        slot0 = it == 0 ? 0 : q;
        if (it > 0) {
            TSVM_LAUNCH(shard_shift_kernel, 1, 1024, 0, st, ids, q, lo, hi, in_ws, m_sd, m_unscale, m_diag);
            TSVM_CUDA(cudaMemcpyAsync(m_hi, (char *) m_hi + (size_t) q * row_bytes, (size_t) q * row_bytes,
                                      cudaMemcpyDeviceToDevice, st));
            TSVM_CUDA(cudaMemcpyAsync(m_lo, (char *) m_lo + (size_t) q * row_bytes, (size_t) q * row_bytes,
                                      cudaMemcpyDeviceToDevice, st));
        }
        // Candidates into the selector's own lists with twice the wanted capacity where it fits (the radix
        // select then stops after two sweeps, see select_fused_kernel), sorted, and the best n_new of every
        // list handed over: the merge of the gathered sorted runs needs no sort.
        const int cap = 2 * n_new <= sel->cand_cap ? 2 * n_new : n_new;
        FusedExtra x;
        x.mode = FUSED_SORT;
        x.sorted_f = cand_f; x.sorted_id = cand_id;
        x.stop = &ctl->stop;
        TSVM_TRY(ws_candidates_cap(sel, kind, n_local, f, alpha, y, it == 0 ? nullptr : in_ws, Cp, Cn, n_new, cap, lo,
                                   sel->cand_f, sel->cand_id, st, x));
        *lists_out = lists;
        *want_out = n_new;
        phase = 1;
        return TSVM_OK;
    }

    // phase B: the same merge on every rank over the gathered lists, then this rank's contributions
    tsvm_status select() {
        TSVM_REQUIRE(phase == 1, "shard solver: phases out of order (select)");
        const int lists = kind == TSVM_SOLVER_C ? 2 : 4;
        const double *mf = all_f;
        const int *mi = all_id;
        if (world > 1) {
            TSVM_LAUNCH(shard_regroup_kernel, ceil_div(world * lists * n_new, 256), 256, 0, st, all_f, all_id, world,
                        lists, n_new, grp_f, grp_id);
            mf = grp_f; mi = grp_id;
        }
        TSVM_TRY(tsvm_ws_merge_sorted(sel, kind, mf, mi, world * n_new, n_new, n_new, ids + slot0, st));
        TSVM_LAUNCH(shard_contrib_kernel, n_new + 4, 256, 0, st, ids, slot0, n_new, ws, lo, hi, km->X, km->ldx, d, dp,
                    km->self_dot, km->diag, y, f, alpha, crow, cstate);
        phase = 2;
        return TSVM_OK;
    }

    // phase C: everything after the exchange, enqueued without waiting. The last launch applies the
    // termination rules on the device (solver_status_kernel); once it has set the stop word, the selection and
    // the local solver of any iteration queued behind it do nothing - the local solver leaves a zero step, so
    // the f updates subtract zero and the scatter writes back the alphas it read.
    tsvm_status enqueue_tail() {
        TSVM_REQUIRE(phase == 2, "shard solver: phases out of order (iterate)");
        TSVM_REQUIRE(queued < MAX_QUEUED, "shard solver: too many iterations queued");
        const long long it = iter + queued;
        const int first_half_phys = (int) (it & 1);
        StepEvents &E = evs[queued];
        if (!E.r0) for (auto e : {&E.r0, &E.r1, &E.b0, &E.b1}) TSVM_CUDA(cudaEventCreate(e));
        TSVM_LAUNCH(shard_unpack_kernel, ceil_div(ws, 256), 256, 0, st, crow, slot0, n_new, dp, ws, cstate, m_sd, m_diag,
                    y_ws, f_ws, a_ws);
        TSVM_TRY(km_stage_rows_features(km, crow, dp + 4, m_sd + slot0, n_new, st));
        TSVM_CUDA(cudaMemcpyAsync((char *) m_hi + (size_t) slot0 * row_bytes, km->Whi, (size_t) n_new * row_bytes,
                                  cudaMemcpyDeviceToDevice, st));
        TSVM_CUDA(cudaMemcpyAsync((char *) m_lo + (size_t) slot0 * row_bytes, km->Wlo, (size_t) n_new * row_bytes,
                                  cudaMemcpyDeviceToDevice, st));
        TSVM_CUDA(cudaMemcpyAsync(m_unscale + slot0, km->w_unscale, sizeof(float) * n_new, cudaMemcpyDeviceToDevice, st));
        TSVM_CUDA(cudaEventRecord(ev_fork, st));
        // second stream: the whole ws x ws block from the members' planes (every rank computes the same
        // values the owners' row buffers hold), then the local solver, replicated
        TSVM_CUDA(cudaStreamWaitEvent(st2, ev_fork, 0));
        const InstancePlanes members{m_hi, m_lo, m_sd, m_unscale, ws};
        const RowPlanes member_rows{m_hi, m_lo, m_sd, m_unscale};
        TSVM_CUDA(cudaEventRecord(E.b0, st2));
        TSVM_TRY(km_rows_planes_on(km, members, member_rows, ws, kww, ws, st2));
        // The kernel-row launch below leaves one SM pair free; started first it would leave the block's eight
        // pairs that one pair to run on, and the local solver - the longer of the two paths once the rows are
        // split - would start late. With iterations queued nothing else orders the two, so the first stream waits
        // for the block.
        TSVM_CUDA(cudaEventRecord(ev_blk, st2));
        TSVM_TRY(launch_local_smo(kind, ws, kww, m_diag, y_ws, f_ws, a_ws, alpha_diff, Cp, Cn, eps, local_max_iter, diff,
                                  nullptr, nullptr, st2, &ctl->stop));
        TSVM_CUDA(cudaEventRecord(E.b1, st2));
        if (it > 0)        // the old half's rows are in the buffer already
            TSVM_LAUNCH(update_f_kernel, update_f_grid(n_local), 128, 0, st2, f, n_local, alpha_diff, ws, q,
                        first_half_phys, rows, ld, rows_vec_ok(rows, ld), 0, q, update_f_cols(n_local), (const int *) nullptr);
        TSVM_CUDA(cudaEventRecord(ev_join, st2));
        // first stream: the new rows against this rank's columns
        float *new_rows = rows + (size_t) (it == 0 ? 0 : (1 - first_half_phys) * q) * ld;
        km->reserve_clusters = 1;
        TSVM_CUDA(cudaStreamWaitEvent(st, ev_blk, 0));
        TSVM_CUDA(cudaEventRecord(E.r0, st));
        const tsvm_status rs = km_rows_staged(km, n_new, new_rows, ld, st);
        km->reserve_clusters = 0;
        TSVM_TRY(rs);
        TSVM_CUDA(cudaEventRecord(E.r1, st));
        TSVM_CUDA(cudaStreamWaitEvent(st, ev_join, 0));
        TSVM_LAUNCH(update_f_kernel, update_f_grid(n_local), 128, 0, st, f, n_local, alpha_diff, ws, q, first_half_phys,
                    rows, ld, rows_vec_ok(rows, ld), it == 0 ? 0 : q, ws, update_f_cols(n_local), (const int *) nullptr);
        TSVM_LAUNCH(shard_scatter_kernel, ceil_div(ws, 256), 256, 0, st, ids, ws, lo, hi, a_ws, alpha);
        TSVM_LAUNCH(solver_status_kernel, 1, 32, 0, st, ctl, diff, sel->count, n_new, eps, -1, (const long long *) nullptr,
                    km->status_dev);
        ++queued;
        phase = 0;
        return TSVM_OK;
    }

    // Waits for the queued iterations and takes over what the device decided (fewer than queued may have run).
    tsvm_status collect() {
        if (queued == 0) return TSVM_OK;
        TSVM_CUDA(cudaMemcpyAsync(ctl_host, ctl, sizeof(SolverCtl), cudaMemcpyDeviceToHost, st));
        TSVM_CUDA(cudaStreamSynchronize(st));
        const SolverCtl &c = *ctl_host;
        const int was_queued = queued;
        queued = 0;
        if (c.engine_status != 0) {
            set_error("dense kernel-row engine reported status %d (a bounded wait ran out)", c.engine_status);
            return TSVM_ERR_DEVICE;
        }
        const int ran = (int) (c.iter - iter);
        for (int j = 0; j < ran && j < was_queued; ++j) {
            float ms_ev = 0;
            cudaEventElapsedTime(&ms_ev, evs[j].r0, evs[j].r1); t_rows += ms_ev;
            cudaEventElapsedTime(&ms_ev, evs[j].b0, evs[j].b1); t_loc += ms_ev;
            rows_made += iter + j == 0 ? ws : q;
        }
        iter = c.iter;
        local_iter = c.local_iter;
        diff0 = c.diff0;
        done = c.done != 0;
        if (c.short_wanted > 0) {
            set_error("working-set selection found %d eligible instances for %d slots (is a class weight or C zero?)",
                      c.short_got, c.short_wanted);
            return TSVM_ERR_INVALID;
        }
        return TSVM_OK;
    }

    tsvm_status iterate() {
        TSVM_TRY(enqueue_tail());
        return collect();
    }

    // One whole outer iteration with the exchange steps enqueued on the solver's stream by the library
    // (needs a communicator): no host work between the phases.
    tsvm_status step() {
        TSVM_REQUIRE(comm || world == 1, "shard solver: tsvm_shard_step needs tsvm_shard_attach_nccl first");
        int lists = 0, want = 0;
        TSVM_TRY(candidates(&lists, &want));
        const size_t m = (size_t) lists * want;
        if (world > 1) {
            NcclApi &nc = nccl_api();
            TSVM_NCCL(nc.GroupStart());
            TSVM_NCCL(nc.AllGather(cand_f, all_f, m, NCCL_FLOAT64, comm, st));
            TSVM_NCCL(nc.AllGather(cand_id, all_id, m, NCCL_INT32, comm, st));
            TSVM_NCCL(nc.GroupEnd());
        } else {
            TSVM_CUDA(cudaMemcpyAsync(all_f, cand_f, m * sizeof(double), cudaMemcpyDeviceToDevice, st));
            TSVM_CUDA(cudaMemcpyAsync(all_id, cand_id, m * sizeof(int), cudaMemcpyDeviceToDevice, st));
        }
        TSVM_TRY(select());
        if (world > 1) {
            NcclApi &nc = nccl_api();
            TSVM_NCCL(nc.GroupStart());
            TSVM_NCCL(nc.AllReduce(crow, crow, (size_t) n_new * (dp + 4), NCCL_FLOAT32, NCCL_SUM, comm, st));
            TSVM_NCCL(nc.AllReduce(cstate, cstate, (size_t) ws * 3, NCCL_FLOAT64, NCCL_SUM, comm, st));
            TSVM_NCCL(nc.GroupEnd());
        }
        return enqueue_tail();
    }

    // Up to n_iters whole iterations, queued sync_every() at a time between reads of the device's verdict.
    tsvm_status run(int n_iters) {
        for (long long end = iter + n_iters; iter < end && !done;) {
            long long k = end - iter;
            if (k > sync_every()) k = sync_every();
            if (iter == 0) k = 1;                   // the first iteration is read back on its own
            for (int j = 0; j < (int) k; ++j) {
                const tsvm_status s = step();
                if (s != TSVM_OK) { collect(); return s; }
            }
            TSVM_TRY(collect());
        }
        return TSVM_OK;
    }
};

extern "C" {

int tsvm_nccl_unique_id(void *id128) {
    NcclApi &nc = nccl_api();
    if (!nc.ok || !id128) { tsvm::set_error("NCCL is not available in this process (libnccl.so.2 not found)"); return TSVM_ERR_INVALID; }
    ncclUniqueIdBytes id;
    const int r = nc.GetUniqueId(&id);
    if (r != 0) { tsvm::set_error("ncclGetUniqueId failed: %s", nc.GetErrorString(r)); return TSVM_ERR_CUDA; }
    memcpy(id128, &id, sizeof(id));
    return TSVM_OK;
}

tsvm_status tsvm_nccl_comm_create(const void *id128, int rank, int world, void **comm_out) {
    TSVM_REQUIRE(id128 && comm_out && world >= 1 && rank >= 0 && rank < world, "nccl_comm_create: bad arguments");
    NcclApi &nc = nccl_api();
    TSVM_REQUIRE(nc.ok, "NCCL is not available in this process (libnccl.so.2 not found)");
    ncclUniqueIdBytes id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    TSVM_NCCL(nc.CommInitRank(&c, world, id, rank));
    *comm_out = c;
    return TSVM_OK;
}

void tsvm_nccl_comm_destroy(void *comm) {
    if (comm && nccl_api().ok) nccl_api().CommDestroy((ncclComm_t) comm);
}

tsvm_status tsvm_shard_attach_nccl(tsvm_shard *S, void *comm) {
    TSVM_REQUIRE(S && comm, "shard_attach_nccl: null argument");
    S->comm = (ncclComm_t) comm;
    return TSVM_OK;
}

tsvm_status tsvm_shard_step(tsvm_shard *S, int *done_host) {
    TSVM_REQUIRE(S && done_host, "shard_step: null argument");
    TSVM_TRY(S->run(1));
    *done_host = S->done ? 1 : 0;
    return TSVM_OK;
}

tsvm_status tsvm_shard_run(tsvm_shard *S, int n_iters, int *done_host) {
    TSVM_REQUIRE(S && n_iters > 0, "shard_run: bad arguments");
    TSVM_TRY(S->run(n_iters));
    if (done_host) *done_host = S->done ? 1 : 0;
    return TSVM_OK;
}

tsvm_status tsvm_shard_create(tsvm_km *km_local, int solver_kind, const int *y_dev, double *alpha_dev, double *f_dev,
                              int n_total, int lo, double eps, double Cp, double Cn, int ws_size, int world,
                              double *cand_f_dev, int *cand_id_dev, double *all_f_dev, int *all_id_dev,
                              float *rows_contrib_dev, double *state_contrib_dev, void *stream, tsvm_shard **out) {
    TSVM_REQUIRE(out && km_local && y_dev && alpha_dev && f_dev && cand_f_dev && cand_id_dev && all_f_dev &&
                 all_id_dev && rows_contrib_dev && state_contrib_dev, "shard_create: null argument");
    TSVM_REQUIRE(solver_kind >= 0 && solver_kind <= 2, "shard_create: unknown solver %d", solver_kind);
    TSVM_REQUIRE(world >= 1 && lo >= 0 && lo + km_local->n <= n_total, "shard_create: bad ownership range");
    TSVM_REQUIRE(ws_size >= 2 && ws_size <= 1024 && ws_size <= n_total && (ws_size & (ws_size - 1)) == 0 &&
                 (long long) world * ws_size <= MERGE_MAX_LEN,
                 "shard_create: working-set size %d must be a power of two in [2, min(n, 1024)] and world * ws <= %d",
                 ws_size, MERGE_MAX_LEN);
    *out = nullptr;
    tsvm_shard *S = new tsvm_shard;
    S->km = km_local; S->kind = solver_kind; S->y = y_dev; S->alpha = alpha_dev; S->f = f_dev;
    S->eps = eps; S->Cp = Cp; S->Cn = Cn; S->ws = ws_size; S->q = ws_size / 2;
    S->n_local = km_local->n; S->n_total = n_total; S->lo = lo; S->hi = lo + km_local->n; S->world = world;
    S->d = km_local->d; S->dp = (km_local->d + 3) & ~3;
    S->ld = ((long long) km_local->n + 3) & ~3ll;
    S->st = (cudaStream_t) stream;
    S->cand_f = cand_f_dev; S->cand_id = cand_id_dev; S->all_f = all_f_dev; S->all_id = all_id_dev;
    S->crow = rows_contrib_dev; S->cstate = state_contrib_dev;
    S->launches0 = launch_count();
    S->t_begin = std::chrono::steady_clock::now();
    tsvm_status s = S->init();
    if (s != TSVM_OK) { delete S; return s; }
    *out = S;
    return TSVM_OK;
}

tsvm_status tsvm_shard_candidates(tsvm_shard *S, int *lists_host, int *want_host) {
    TSVM_REQUIRE(S && lists_host && want_host, "shard_candidates: null argument");
    return S->candidates(lists_host, want_host);
}

tsvm_status tsvm_shard_select(tsvm_shard *S, int *n_new_host) {
    TSVM_REQUIRE(S && n_new_host, "shard_select: null argument");
    TSVM_TRY(S->select());
    *n_new_host = S->n_new;
    return TSVM_OK;
}

tsvm_status tsvm_shard_iterate(tsvm_shard *S, int *done_host) {
    TSVM_REQUIRE(S && done_host, "shard_iterate: null argument");
    TSVM_TRY(S->iterate());
    *done_host = S->done ? 1 : 0;
    return TSVM_OK;
}

tsvm_status tsvm_shard_get_stats(const tsvm_shard *S, tsvm_solve_stats *out) {
    TSVM_REQUIRE(S && out, "shard_get_stats: null argument");
    memset(out, 0, sizeof(*out));
    out->outer_iters = S->iter;
    out->local_iters = S->local_iter;
    out->final_diff = S->diff0;
    out->objective = NAN;
    out->seconds_rows = S->t_rows * 1e-3;
    out->seconds_local = S->t_loc * 1e-3;       // ws x ws block + local solver, on the second stream
    out->seconds_total = std::chrono::duration<double>(std::chrono::steady_clock::now() - S->t_begin).count();
    out->kernel_rows = S->rows_made;
    out->gpu_launches = launch_count() - S->launches0;
    return TSVM_OK;
}

void tsvm_shard_destroy(tsvm_shard *S) { delete S; }

}  // extern "C"
