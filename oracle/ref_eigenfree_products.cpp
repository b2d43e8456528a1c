// TEST INFRASTRUCTURE ONLY - never linked into or called by the product library.
//
// Eigen-free stand-ins for the four svm_kernel:: symbols that the reference's CPU
// backend cannot provide in this image:
//   * dns_csr_mul, csr_csr_mul, dns_dns_mul  - the reference implements them with
//     Eigen (src/thundersvm/kernel/kernelmatrix_kernel.cpp:149-187); Eigen is an
//     un-vendored git submodule (.gitmodules:1-3, empty eigen/ directory, no
//     pinned tag; CMakeLists.txt:45 accepts any Eigen >= 3.3) and absent here.
//   * sum_kernel_values_instant - declared in
//     include/thundersvm/kernel/kernelmatrix_kernel.h:42-45, defined only in the
//     CUDA backend (src/thundersvm/kernel/kernelmatrix_kernel.cu:99-138,164-172).
// Every other reference translation unit is compiled unmodified from its own
// source tree by oracle/Makefile.
//
// Arithmetic restated: Eigen 3.3's row-major-sparse x dense product evaluates, for
// every output coefficient, "tmp = 0; for each stored entry of the sparse row in
// storage order: tmp += value * rhs(col, c)" in the scalar type (float), then
// stores tmp. That per-coefficient recurrence is what the loops below perform.
#include <thundersvm/kernel/kernelmatrix_kernel.h>
#include <cstdio>
#include <cstdlib>

namespace svm_kernel {

    // result(m x n, column-major: result[c*m + i]) = CSR(m x k) * dense_mat(k x n
    // column-major, i.e. the n working-set rows stored row-major with stride k).
    // Follows kernelmatrix_kernel.cpp:149-160.
    void dns_csr_mul(int m, int n, int k, const SyncArray<kernel_type> &dense_mat,
                     const SyncArray<kernel_type> &csr_val, const SyncArray<int> &csr_row_ptr,
                     const SyncArray<int> &csr_col_ind, int nnz, SyncArray<kernel_type> &result) {
        (void) nnz;
        const kernel_type *B = dense_mat.host_data();
        const kernel_type *val = csr_val.host_data();
        const int *rp = csr_row_ptr.host_data();
        const int *ci = csr_col_ind.host_data();
        kernel_type *out = result.host_data();
#pragma omp parallel for schedule(guided)
        for (int i = 0; i < m; ++i) {
            const int b = rp[i], e = rp[i + 1];
            for (int c = 0; c < n; ++c) {
                const kernel_type *col = B + (size_t) c * k;
                kernel_type t = 0;
                for (int p = b; p < e; ++p) t += val[p] * col[ci[p]];
                out[(size_t) c * m + i] = t;
            }
        }
    }

    // result(m x n, column-major) = CSR1(m x k) * CSC2(k x n); CSC2's columns are the
    // working-set rows. Follows kernelmatrix_kernel.cpp:162-176. Both index lists are
    // ascending within a row, so a merge-join visits the common columns in order.
    void csr_csr_mul(int m, int n, int k, const SyncArray<kernel_type> &ws_val, const SyncArray<int> &ws_col_ind,
                     const SyncArray<int> &ws_row_ptr, const SyncArray<kernel_type> &csr_val,
                     const SyncArray<int> &csr_row_ptr, const SyncArray<int> &csr_col_ind, int nnz, int nnz2,
                     SyncArray<kernel_type> &result) {
        (void) k; (void) nnz; (void) nnz2;
        const kernel_type *v2 = ws_val.host_data();
        const int *c2 = ws_col_ind.host_data();
        const int *p2 = ws_row_ptr.host_data();
        const kernel_type *v1 = csr_val.host_data();
        const int *p1 = csr_row_ptr.host_data();
        const int *c1 = csr_col_ind.host_data();
        kernel_type *out = result.host_data();
#pragma omp parallel for schedule(guided)
        for (int i = 0; i < m; ++i) {
            for (int c = 0; c < n; ++c) {
                int a = p1[i], ae = p1[i + 1], b = p2[c], be = p2[c + 1];
                kernel_type t = 0;
                while (a < ae && b < be) {
                    if (c1[a] == c2[b]) t += v1[a++] * v2[b++];
                    else if (c1[a] < c2[b]) ++a;
                    else ++b;
                }
                out[(size_t) c * m + i] = t;
            }
        }
    }

    // result(m x n, column-major) = origin_dense(m x k row-major) * dense_mat(k x n
    // column-major). Follows kernelmatrix_kernel.cpp:178-187 (not reached by any
    // reference call path in the CPU build; kept so the link is complete).
    void dns_dns_mul(int m, int n, int k, const SyncArray<kernel_type> &dense_mat,
                     const SyncArray<kernel_type> &origin_dense, SyncArray<kernel_type> &result) {
        const kernel_type *B = dense_mat.host_data();
        const kernel_type *A = origin_dense.host_data();
        kernel_type *out = result.host_data();
#pragma omp parallel for schedule(guided)
        for (int i = 0; i < m; ++i)
            for (int c = 0; c < n; ++c) {
                kernel_type t = 0;
                for (int p = 0; p < k; ++p) t += A[(size_t) i * k + p] * B[(size_t) c * k + p];
                out[(size_t) c * m + i] = t;
            }
    }

    // CUDA-only entry points of the reference (kernelmatrix_kernel.cpp:188-196 prints
    // "No implementing..." for them); never reached by the CPU call paths.
    void dns_dns_mul(int, int, int, const SyncArray<kernel_type> &, const SyncArray<kernel_type> &, kernel_type,
                     SyncArray<kernel_type> &) {
        fprintf(stderr, "dns_dns_mul(beta): CUDA-only symbol reached in the CPU oracle\n");
        abort();
    }

    void get_working_set_ins_dns(const SyncArray<kernel_type> &, const SyncArray<int> &, SyncArray<kernel_type> &,
                                 int, int, int) {
        fprintf(stderr, "get_working_set_ins_dns: CUDA-only symbol reached in the CPU oracle\n");
        abort();
    }

    // Decision values + one-vs-one vote on the spot. Follows
    // kernelmatrix_kernel.cu:99-138 (one test row per loop trip).
    void sum_kernel_values_instant(const SyncArray<float_type> &coef, int total_sv, const SyncArray<int> &sv_start,
                                   const SyncArray<int> &sv_count, const SyncArray<float_type> &rho,
                                   const SyncArray<kernel_type> &k_mat, SyncArray<float_type> &predict_instant,
                                   int n_classes, int n_instances, SyncArray<float_type> &vote_device) {
        const float_type *cf = coef.host_data();
        const int *ss = sv_start.host_data();
        const int *sc = sv_count.host_data();
        const float_type *r = rho.host_data();
        const kernel_type *K = k_mat.host_data();
        float_type *pred = predict_instant.host_data();
        float_type *vote = vote_device.host_data();
#pragma omp parallel for schedule(guided)
        for (int idx = 0; idx < n_instances; ++idx) {
            float_type *v = vote + (size_t) idx * n_classes;
            for (int i = 0; i < n_classes; ++i) v[i] = 0;
            size_t kk = 0;
            const kernel_type *kv = K + (size_t) idx * total_sv;
            for (int i = 0; i < n_classes; ++i)
                for (int j = i + 1; j < n_classes; ++j) {
                    const float_type *c1 = cf + (size_t) (j - 1) * total_sv;
                    const float_type *c2 = cf + (size_t) i * total_sv;
                    double sum = 0;
                    for (int l = 0; l < sc[i]; ++l) sum += c1[ss[i] + l] * kv[ss[i] + l];
                    for (int l = 0; l < sc[j]; ++l) sum += c2[ss[j] + l] * kv[ss[j] + l];
                    if (sum - r[kk] > 0) v[i]++; else v[j]++;
                    kk++;
                }
            int best = 0;
            for (int i = 1; i < n_classes; ++i) if (v[i] > v[best]) best = i;
            pred[idx] = best;
        }
    }
}
