/* TEST INFRASTRUCTURE ONLY - CPU restatement ("port") of the reference algorithm for
 * the batched-SMO hot path. Built into oracle/libsvm_oracle.so by oracle/Makefile and
 * loaded only by tests/, the smoke check and the benchmark's CPU-baseline leg, as the
 * checker. The product library never links, loads or calls it.
 *
 * Parity status: PINNED. The restatement is checked (tests/test_oracle.py) against
 *   - the reference's own CPU objects compiled from its sources (oracle/_ref), and
 *   - the committed fixtures under tests/golden/ generated from that build, including
 *     the reference tests' known answers on dataset/test_dataset.txt
 *     (src/test/test_svc.cpp:36, test_nusvc.cpp:43, test_svr.cpp:38, test_nusvr.cpp:41,
 *      test_oneclass_svc.cpp:27, test_kernelmatrix.cpp:123-143).
 *
 * Types follow include/thundersvm/thundersvm.h:16-22: float_type = double (alpha, f,
 * rho, coef, decision values), kernel_type = float (feature values, kernel values,
 * self dots). Data is CSR with the column ids the caller uses (the reference keeps
 * LibSVM's 1-based ids; any consistent numbering gives the same dot products).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

enum { K_LINEAR = 0, K_POLY = 1, K_RBF = 2, K_SIGMOID = 3, K_PRECOMPUTED = 4 };

typedef struct {
    int n, n_features;          /* n_features = max column id + 1 (kernelmatrix.cpp:200-206) */
    const float *val;
    const int *row_ptr, *col;
    int kernel;
    int degree;
    float gamma, coef0;
} csr_t;

static int is_I_up(double a, double y, double Cp, double Cn) {   /* smo_kernel.h:13-15 */
    (void) Cn;
    return (y > 0 && a < Cp) || (y < 0 && a > 0);
}

static int is_I_low(double a, double y, double Cp, double Cn) {  /* smo_kernel.h:17-19 */
    (void) Cp;
    return (y > 0 && a > 0) || (y < 0 && a < Cn);
}

static int is_free(double a, double y, double Cp, double Cn) {   /* smo_kernel.h:21-23 */
    return a > 0 && (y > 0 ? a < Cp : a < Cn);
}

/* self dots: double accumulation, float store (kernelmatrix.cpp:194-204) */
void oracle_self_dot(int n, const float *val, const int *row_ptr, float *out) {
    for (int i = 0; i < n; ++i) {
        double s = 0;
        for (int p = row_ptr[i]; p < row_ptr[i + 1]; ++p) s += val[p] * val[p];
        out[i] = (float) s;
    }
}

/* diagonal K(x_i, x_i) (kernelmatrix.cpp:225-247) */
void oracle_diag(int n, const float *val, const int *row_ptr, int kernel, int degree, float gamma, float coef0,
                 float *out) {
    oracle_self_dot(n, val, row_ptr, out);
    for (int i = 0; i < n; ++i) {
        switch (kernel) {
            case K_RBF: case K_PRECOMPUTED: out[i] = 1; break;
            case K_LINEAR: break;
            case K_POLY: out[i] = powf(gamma * out[i] + coef0, degree); break;
            case K_SIGMOID: out[i] = tanhf(gamma * out[i] + coef0); break;
        }
    }
}

static void transform_rows(float *rows, int m, int n, const float *sd_rows, const float *sd_all, int kernel,
                           int degree, float gamma, float coef0) {
    /* kernelmatrix_kernel.cpp:61-108 */
#pragma omp parallel for schedule(guided)
    for (int i = 0; i < m; ++i) {
        float *r = rows + (size_t) i * n;
        switch (kernel) {
            case K_RBF: case K_PRECOMPUTED:
                for (int j = 0; j < n; ++j) r[j] = expf(-(sd_rows[i] + sd_all[j] - r[j] * 2) * gamma);
                break;
            case K_POLY:
                for (int j = 0; j < n; ++j) r[j] = powf(gamma * r[j] + coef0, degree);
                break;
            case K_SIGMOID:
                for (int j = 0; j < n; ++j) r[j] = tanhf(gamma * r[j] + coef0);
                break;
            default: break;
        }
    }
}

/* out[c*n + i] = sum over the stored entries p of instance i, in storage order, of
 * val[p] * B[c][col[p]] with float accumulation: the per-coefficient recurrence of the
 * reference's sparse(row-major) x dense product (kernelmatrix_kernel.cpp:149-160). */
static void dns_csr_mul(const csr_t *X, const float *B, int m, float *out) {
    const int n = X->n, k = X->n_features;
#pragma omp parallel for schedule(guided)
    for (int i = 0; i < n; ++i) {
        const int b = X->row_ptr[i], e = X->row_ptr[i + 1];
        for (int c = 0; c < m; ++c) {
            const float *row = B + (size_t) c * k;
            float t = 0;
            for (int p = b; p < e; ++p) t += X->val[p] * row[X->col[p]];
            out[(size_t) c * n + i] = t;
        }
    }
}

/* KernelMatrix::get_rows(idx) (kernelmatrix.cpp:251-279 via :378-383): densify the
 * chosen rows (row-major, m x n_features), product, kernel transform. */
static void get_rows_idx(const csr_t *X, const float *self_dot, const int *idx, int m, float *out) {
    const int k = X->n_features;
    float *B = (float *) calloc((size_t) m * k, sizeof(float));
    float *sd = (float *) malloc(sizeof(float) * m);
    for (int c = 0; c < m; ++c) {
        const int r = idx[c];
        for (int p = X->row_ptr[r]; p < X->row_ptr[r + 1]; ++p) B[(size_t) c * k + X->col[p]] = X->val[p];
        sd[c] = self_dot[r];
    }
    dns_csr_mul(X, B, m, out);
    transform_rows(out, m, X->n, sd, self_dot, X->kernel, X->degree, X->gamma, X->coef0);
    free(B);
    free(sd);
}

void oracle_kernel_rows_idx(int n, int n_features, const float *val, const int *row_ptr, const int *col, int kernel,
                            int degree, float gamma, float coef0, const int *idx, int m, float *out) {
    csr_t X = {n, n_features, val, row_ptr, col, kernel, degree, gamma, coef0};
    float *sd = (float *) malloc(sizeof(float) * n);
    oracle_self_dot(n, val, row_ptr, sd);
    get_rows_idx(&X, sd, idx, m, out);
    free(sd);
}

/* KernelMatrix::get_rows(instances) (kernelmatrix.cpp:281-312, :385-406): features
 * with id >= n_features are dropped from the product but NOT from the test self dot,
 * which is accumulated in float. */
void oracle_kernel_rows_ins(int n, int n_features, const float *val, const int *row_ptr, const int *col, int kernel,
                            int degree, float gamma, float coef0, int m, const float *tval, const int *trow_ptr,
                            const int *tcol, float *out) {
    csr_t X = {n, n_features, val, row_ptr, col, kernel, degree, gamma, coef0};
    float *sd = (float *) malloc(sizeof(float) * n);
    oracle_self_dot(n, val, row_ptr, sd);
    float *B = (float *) calloc((size_t) m * n_features, sizeof(float));
    float *tsd = (float *) malloc(sizeof(float) * m);
    for (int c = 0; c < m; ++c) {
        float s = 0;
        for (int p = trow_ptr[c]; p < trow_ptr[c + 1]; ++p) {
            if (tcol[p] < n_features) B[(size_t) c * n_features + tcol[p]] = tval[p];
            s = fmaf(tval[p], tval[p], s);   /* the reference's Release build fuses this (FMA targets) */
        }
        tsd[c] = s;
    }
    dns_csr_mul(&X, B, m, out);
    transform_rows(out, m, n, tsd, sd, kernel, degree, gamma, coef0);
    free(B);
    free(tsd);
    free(sd);
}

/* ---- local solvers -------------------------------------------------------------- */

/* c_smo_solve_kernel, CPU form (smo_kernel.cpp:12-125). Ties go to the lowest slot. */
static void c_smo_local(const int *label, const double *f_val, double *alpha, double *alpha_diff, const int *ws,
                        int ws_size, double Cp, double Cn, const float *rows, const float *diag, int row_len,
                        double eps, double *diff, int max_iter) {
    double *a_old = malloc(sizeof(double) * ws_size), *a = malloc(sizeof(double) * ws_size);
    double *f = malloc(sizeof(double) * ws_size), *y = malloc(sizeof(double) * ws_size);
    double *kI = malloc(sizeof(double) * ws_size);
    float *kd = malloc(sizeof(float) * ws_size);
    for (int t = 0; t < ws_size; ++t) {
        int w = ws[t];
        f[t] = f_val[w];
        a_old[t] = a[t] = alpha[w];
        y[t] = label[w];
        kd[t] = diag[w];
    }
    double local_eps = 0;
    int it = 0;
    for (;;) {
        int i = 0;
        double up = INFINITY;
        for (int t = 0; t < ws_size; ++t)
            if (is_I_up(a[t], y[t], Cp, Cn) && f[t] < up) { up = f[t]; i = t; }
        for (int t = 0; t < ws_size; ++t) kI[t] = rows[(size_t) row_len * i + ws[t]];
        double low = -INFINITY;
        for (int t = 0; t < ws_size; ++t)
            if (is_I_low(a[t], y[t], Cp, Cn) && f[t] > low) low = f[t];
        double local_diff = low - up;
        if (it == 0) {
            local_eps = fmax(eps, 0.1f * local_diff);   /* 0.1f promoted, smo_kernel.cpp:64 */
            diff[0] = local_diff;
        }
        if (it > max_iter || local_diff < local_eps) {
            for (int t = 0; t < ws_size; ++t) {
                alpha_diff[t] = -(a[t] - a_old[t]) * y[t];
                alpha[ws[t]] = a[t];
            }
            diff[1] = it;
            break;
        }
        int j2 = 0;
        double min_t = INFINITY;
        for (int t = 0; t < ws_size; ++t)
            if (-up > -f[t] && is_I_low(a[t], y[t], Cp, Cn)) {
                double aIJ = kd[i] + kd[t] - 2 * kI[t];
                double bIJ = -up + f[t];
                double ft = -bIJ * bIJ / aIJ;
                if (ft < min_t) { min_t = ft; j2 = t; }
            }
        double di = y[i] > 0 ? Cp - a[i] : a[i];
        double dj = fmin(y[j2] > 0 ? a[j2] : Cn - a[j2], (-up + f[j2]) / (kd[i] + kd[j2] - 2 * kI[j2]));
        double l = fmin(di, dj);
        a[i] += l * y[i];
        a[j2] -= l * y[j2];
        for (int t = 0; t < ws_size; ++t) {
            double kJ = rows[(size_t) row_len * j2 + ws[t]];
            f[t] -= l * (kJ - kI[t]);
        }
        it++;
    }
    free(a_old); free(a); free(f); free(y); free(kI); free(kd);
}

/* nu_smo_solve_kernel. cuda_semantics = 0 follows the CPU backend (smo_kernel.cpp:127-298:
 * the negative-class second-order pick uses kd[ip] and K[ip,.], diff[1] is never written);
 * cuda_semantics = 1 follows the CUDA backend (smo_kernel.cu:118-252: kd[in] and K[in,.],
 * bound C held in float, diff[1] = #iterations). */
static void nu_smo_local(const int *label, const double *f_val, double *alpha, double *alpha_diff, const int *ws,
                         int ws_size, double C_in, const float *rows, const float *diag, int row_len, double eps,
                         double *diff, int max_iter, int cuda_semantics) {
    const double C = cuda_semantics ? (double) (float) C_in : C_in;
    double *a_old = malloc(sizeof(double) * ws_size), *a = malloc(sizeof(double) * ws_size);
    double *f = malloc(sizeof(double) * ws_size);
    int *y = malloc(sizeof(int) * ws_size);
    float *kIp = malloc(sizeof(float) * ws_size), *kIn = malloc(sizeof(float) * ws_size);
    float *kd = malloc(sizeof(float) * ws_size);
    for (int t = 0; t < ws_size; ++t) {
        int w = ws[t];
        f[t] = f_val[w];
        a_old[t] = a[t] = alpha[w];
        y[t] = label[w];
        kd[t] = diag[w];
    }
    double local_eps = 0;
    int it = 0;
    for (;;) {
        int ip = 0, in = 0;
        double up_p = INFINITY, up_n = INFINITY, low_p = -INFINITY, low_n = -INFINITY;
        for (int t = 0; t < ws_size; ++t)
            if (y[t] > 0 && a[t] < C && f[t] < up_p) { ip = t; up_p = f[t]; }
        for (int t = 0; t < ws_size; ++t) kIp[t] = rows[(size_t) row_len * ip + ws[t]];
        for (int t = 0; t < ws_size; ++t)
            if (y[t] < 0 && a[t] > 0 && f[t] < up_n) { in = t; up_n = f[t]; }
        for (int t = 0; t < ws_size; ++t) kIn[t] = rows[(size_t) row_len * in + ws[t]];
        for (int t = 0; t < ws_size; ++t)
            if (y[t] > 0 && a[t] > 0 && f[t] > low_p) low_p = f[t];
        for (int t = 0; t < ws_size; ++t)
            if (y[t] < 0 && a[t] < C && f[t] > low_n) low_n = f[t];
        double local_diff = fmax(low_p - up_p, low_n - up_n);
        if (it == 0) {
            local_eps = fmax(eps, 0.1 * local_diff);
            diff[0] = local_diff;
        }
        if (it > max_iter || local_diff < local_eps) {
            for (int t = 0; t < ws_size; ++t) {
                alpha_diff[t] = -(a[t] - a_old[t]) * y[t];
                alpha[ws[t]] = a[t];
            }
            if (cuda_semantics) diff[1] = it;
            break;
        }
        int j2p = 0, j2n = 0;
        double vp = INFINITY, vn = INFINITY;
        for (int t = 0; t < ws_size; ++t)
            if (-up_p > -f[t] && y[t] > 0 && a[t] > 0) {
                double aIJ = kd[ip] + kd[t] - 2 * kIp[t];
                double bIJ = -up_p + f[t];
                double v = -bIJ * bIJ / aIJ;
                if (v < vp) { j2p = t; vp = v; }
            }
        for (int t = 0; t < ws_size; ++t)
            if (-up_n > -f[t] && y[t] < 0 && a[t] < C) {
                double aIJ = cuda_semantics ? kd[in] + kd[t] - 2 * kIn[t] : kd[ip] + kd[t] - 2 * kIp[t];
                double bIJ = -up_n + f[t];
                double v = -bIJ * bIJ / aIJ;
                if (v < vn) { j2n = t; vn = v; }
            }
        int i, j2;
        double up;
        const float *kI;
        if (vp < vn) { i = ip; j2 = j2p; up = up_p; kI = kIp; }
        else { i = in; j2 = j2n; up = up_n; kI = kIn; }
        double di = y[i] > 0 ? C - a[i] : a[i];
        double dj = fmin(y[j2] > 0 ? a[j2] : C - a[j2], (-up + f[j2]) / (kd[i] + kd[j2] - 2 * kI[j2]));
        double l = fmin(di, dj);
        a[i] += l * y[i];
        a[j2] -= l * y[j2];
        for (int t = 0; t < ws_size; ++t) {
            float kJ = rows[(size_t) row_len * j2 + ws[t]];
            f[t] -= l * (kJ - kI[t]);
        }
        it++;
    }
    free(a_old); free(a); free(f); free(y); free(kIp); free(kIn); free(kd);
}

void oracle_local_smo(int solver_kind, int cuda_semantics, const int *label, const double *f_val, double *alpha,
                      double *alpha_diff, const int *ws, int ws_size, double Cp, double Cn, const float *rows,
                      const float *diag, int row_len, double eps, double *diff, int max_iter) {
    if (solver_kind == 0) c_smo_local(label, f_val, alpha, alpha_diff, ws, ws_size, Cp, Cn, rows, diag, row_len, eps,
                                      diff, max_iter);
    else nu_smo_local(label, f_val, alpha, alpha_diff, ws, ws_size, Cp, rows, diag, row_len, eps, diff, max_iter,
                      cuda_semantics);
}

/* update_f (smo_kernel.cpp:300-319) */
void oracle_update_f(double *f, int n, const double *alpha_diff, int m, const float *rows) {
#pragma omp parallel for schedule(guided)
    for (int j = 0; j < n; ++j) {
        double s = 0;
        for (int i = 0; i < m; ++i) {
            double d = alpha_diff[i];
            if (d != 0) s += d * rows[(size_t) i * n + j];
        }
        f[j] -= s;
    }
}

/* sort_f (smo_kernel.cpp:321-332): ascending by (f, index). */
typedef struct { double f; int i; } fi_t;
static int fi_cmp(const void *pa, const void *pb) {
    const fi_t *a = pa, *b = pb;
    if (a->f < b->f) return -1;
    if (a->f > b->f) return 1;
    return (a->i > b->i) - (a->i < b->i);
}

/* CSMOSolver::select_working_set (csmosolver.cpp:123-165) */
static void select_ws_c(int n, char *ind, const int *order, const int *y, const double *alpha, double Cp, double Cn,
                        int *out, int want) {
    int pl = 0, pr = n - 1, got = 0;
    while (got < want) {
        int i;
        if (pl < n) {
            i = order[pl];
            while (ind[i] || !is_I_up(alpha[i], y[i], Cp, Cn)) {
                if (++pl == n) break;
                i = order[pl];
            }
            if (pl < n) { out[got++] = i; ind[i] = 1; }
        }
        if (pr >= 0) {
            i = order[pr];
            while (ind[i] || !is_I_low(alpha[i], y[i], Cp, Cn)) {
                if (--pr == -1) break;
                i = order[pr];
            }
            if (pr >= 0) { out[got++] = i; ind[i] = 1; }
        }
        if (pl >= n && pr < 0) break;   /* the reference would spin here; cannot happen for ws <= n */
    }
}

/* NuSMOSolver::select_working_set (nusmosolver.cpp:48-118) */
static void select_ws_nu(int n, char *ind, const int *order, const int *y, const double *alpha, double Cp, double Cn,
                         int *out, int want) {
    int plp = 0, pln = 0, prp = n - 1, prn = n - 1, got = 0;
    while (got < want) {
        int i;
        if (plp < n) {
            i = order[plp];
            while (ind[i] || !(y[i] > 0 && is_I_up(alpha[i], y[i], Cp, Cn))) {
                if (++plp == n) break;
                i = order[plp];
            }
            if (plp < n) { out[got++] = i; ind[i] = 1; }
        }
        if (pln < n) {
            i = order[pln];
            while (ind[i] || !(y[i] < 0 && is_I_up(alpha[i], y[i], Cp, Cn))) {
                if (++pln == n) break;
                i = order[pln];
            }
            if (pln < n && got < want) { out[got++] = i; ind[i] = 1; }
        }
        if (prp >= 0) {
            i = order[prp];
            while (ind[i] || !(y[i] > 0 && is_I_low(alpha[i], y[i], Cp, Cn))) {
                if (--prp == -1) break;
                i = order[prp];
            }
            if (prp >= 0 && got < want) { out[got++] = i; ind[i] = 1; }
        }
        if (prn >= 0) {
            i = order[prn];
            while (ind[i] || !(y[i] < 0 && is_I_low(alpha[i], y[i], Cp, Cn))) {
                if (--prn == -1) break;
                i = order[prn];
            }
            if (prn >= 0 && got < want) { out[got++] = i; ind[i] = 1; }
        }
        if (plp >= n && pln >= n && prp < 0 && prn < 0) break;
    }
}

/* Working-set selection alone, for unit tests: in_ws[n] marks instances already held. */
void oracle_select_working_set(int solver_kind, int n, const double *f, const int *y, const double *alpha, double Cp,
                               double Cn, const char *in_ws, int *out, int want) {
    fi_t *s = malloc(sizeof(fi_t) * n);
    int *order = malloc(sizeof(int) * n);
    char *ind = malloc(n);
    for (int i = 0; i < n; ++i) { s[i].f = f[i]; s[i].i = i; ind[i] = in_ws ? in_ws[i] : 0; }
    qsort(s, n, sizeof(fi_t), fi_cmp);
    for (int i = 0; i < n; ++i) order[i] = s[i].i;
    if (solver_kind == 0) select_ws_c(n, ind, order, y, alpha, Cp, Cn, out, want);
    else select_ws_nu(n, ind, order, y, alpha, Cp, Cn, out, want);
    free(s); free(order); free(ind);
}

/* calculate_rho (csmosolver.cpp:167-187) */
static double rho_c(int n, const double *f, const int *y, const double *alpha, double Cp, double Cn) {
    int n_free = 0;
    double sum = 0, up = INFINITY, low = -INFINITY;
    for (int i = 0; i < n; ++i) {
        if (is_free(alpha[i], y[i], Cp, Cn)) { n_free++; sum += f[i]; }
        if (is_I_up(alpha[i], y[i], Cp, Cn)) up = fmin(up, f[i]);
        if (is_I_low(alpha[i], y[i], Cp, Cn)) low = fmax(low, f[i]);
    }
    return n_free ? sum / n_free : -(up + low) / 2;
}

/* NuSMOSolver::calculate_rho + scale_alpha_rho (nusmosolver.cpp:9-46,120-126) */
static double rho_nu(int n, const double *f, const int *y, double *alpha, double Cp, double Cn, int for_svr) {
    int nfp = 0, nfn = 0;
    double sp = 0, sn = 0, up_p = INFINITY, up_n = INFINITY, low_p = -INFINITY, low_n = -INFINITY;
    for (int i = 0; i < n; ++i) {
        if (y[i] > 0) {
            if (alpha[i] > 0 && alpha[i] < Cp) { nfp++; sp += f[i]; }
            if (is_I_up(alpha[i], y[i], Cp, Cn)) up_p = fmin(up_p, -f[i]);
            if (is_I_low(alpha[i], y[i], Cp, Cn)) low_p = fmax(low_p, -f[i]);
        } else {
            if (alpha[i] > 0 && alpha[i] < Cn) { nfn++; sn += -f[i]; }
            if (is_I_up(alpha[i], y[i], Cp, Cn)) up_n = fmin(up_n, -f[i]);
            if (is_I_low(alpha[i], y[i], Cp, Cn)) low_n = fmax(low_n, -f[i]);
        }
    }
    double r1 = nfp ? sp / nfp : -(up_p + low_p) / 2;
    double r2 = nfn ? sn / nfn : -(up_n + low_n) / 2;
    double rho = (r1 - r2) / 2;
    if (!for_svr) {
        double r = (r1 + r2) / 2;
        for (int i = 0; i < n; ++i) alpha[i] /= r;
        rho /= r;
    }
    return rho;
}

/* calculate_obj (csmosolver.cpp:227-239) */
double oracle_objective(int n, const double *f, const double *alpha, const int *y) {
    double obj = 0;
    for (int i = 0; i < n; ++i) obj += alpha[i] - (f[i] + y[i]) * alpha[i] * y[i] / 2;
    return -obj;
}

/* CSMOSolver::solve (csmosolver.cpp:10-121) with init_f (:189-214).
 * solver_kind: 0 = C-SMO, 1 = nu-SMO for nu-SVC (alpha/rho scaled), 2 = nu-SMO for nu-SVR.
 * stats[0] = outer iterations run, [1] = total local iterations, [2] = last diff[0],
 * stats[3] = objective before any nu scaling. ws_trace (may be NULL) receives the first
 * trace_iters working sets, ws_size ids each. */
void oracle_smo_solve(int n, int n_features, const float *val, const int *row_ptr, const int *col, int kernel,
                      int degree, float gamma, float coef0, int solver_kind, int cuda_semantics, const int *y,
                      double *alpha, double *f_val, double eps, double Cp, double Cn, int ws_size, int out_max_iter,
                      double *rho_out, double *stats, int *ws_trace, int trace_iters) {
    csr_t X = {n, n_features, val, row_ptr, col, kernel, degree, gamma, coef0};
    const int q = ws_size / 2;
    float *sd = malloc(sizeof(float) * n), *diag = malloc(sizeof(float) * n);
    oracle_self_dot(n, val, row_ptr, sd);
    oracle_diag(n, val, row_ptr, kernel, degree, gamma, coef0, diag);
    int *ws = malloc(sizeof(int) * ws_size), *order = malloc(sizeof(int) * n);
    char *ind = malloc(n);
    fi_t *srt = malloc(sizeof(fi_t) * n);
    double *alpha_diff = malloc(sizeof(double) * ws_size);
    float *rows = malloc(sizeof(float) * (size_t) ws_size * n);
    double diff[2] = {0, 0};

    /* init_f: batches of 101 non-zero alphas */
    {
        int cap = 101, cnt = 0;
        int *bidx = malloc(sizeof(int) * cap);
        double *bd = malloc(sizeof(double) * cap);
        float *brows = NULL;
        for (int i = 0; i < n; ++i) {
            if (alpha[i] != 0) { bidx[cnt] = i; bd[cnt] = -alpha[i] * y[i]; cnt++; }
            if (cnt > 100 || (i == n - 1 && cnt > 0)) {
                if (!brows) brows = malloc(sizeof(float) * (size_t) cap * n);
                get_rows_idx(&X, sd, bidx, cnt, brows);
                oracle_update_f(f_val, n, bd, cnt, brows);
                cnt = 0;
            }
        }
        free(bidx); free(bd); free(brows);
    }

    int max_iter = ws_size > 2147483647 / 100 ? 2147483647 : 100 * ws_size;
    if (max_iter < 100000) max_iter = 100000;
    long long local_iter = 0;
    int same_cnt = 0, swap_cnt = 0;
    double prev = INFINITY, last = INFINITY, second_last = INFINITY;
    int iter;
    for (iter = 0;; ++iter) {
        for (int i = 0; i < n; ++i) { srt[i].f = f_val[i]; srt[i].i = i; }
        qsort(srt, n, sizeof(fi_t), fi_cmp);
        for (int i = 0; i < n; ++i) order[i] = srt[i].i;
        memset(ind, 0, n);
        if (iter == 0) {
            if (solver_kind == 0) select_ws_c(n, ind, order, y, alpha, Cp, Cn, ws, ws_size);
            else select_ws_nu(n, ind, order, y, alpha, Cp, Cn, ws, ws_size);
            get_rows_idx(&X, sd, ws, ws_size, rows);
        } else {
            memcpy(ws, ws + q, sizeof(int) * q);
            for (int i = 0; i < q; ++i) ind[ws[i]] = 1;
            if (solver_kind == 0) select_ws_c(n, ind, order, y, alpha, Cp, Cn, ws + q, q);
            else select_ws_nu(n, ind, order, y, alpha, Cp, Cn, ws + q, q);
            memcpy(rows, rows + (size_t) q * n, sizeof(float) * (size_t) q * n);
            get_rows_idx(&X, sd, ws + q, q, rows + (size_t) q * n);
        }
        if (ws_trace && iter < trace_iters) memcpy(ws_trace + (size_t) iter * ws_size, ws, sizeof(int) * ws_size);
        if (solver_kind == 0) c_smo_local(y, f_val, alpha, alpha_diff, ws, ws_size, Cp, Cn, rows, diag, n, eps, diff,
                                          max_iter);
        else nu_smo_local(y, f_val, alpha, alpha_diff, ws, ws_size, Cp, rows, diag, n, eps, diff, max_iter,
                          cuda_semantics);
        oracle_update_f(f_val, n, alpha_diff, ws_size, rows);
        local_iter += (long long) diff[1];
        if (fabs(diff[0] - prev) < eps * 0.001) same_cnt++;
        else { same_cnt = 0; prev = diff[0]; }
        if (fabs(diff[0] - second_last) < eps * 0.001) swap_cnt++;
        else swap_cnt = 0;
        second_last = last;
        last = diff[0];
        if ((same_cnt >= 10 && fabs(diff[0] - 2.0) > eps) || diff[0] < eps ||
            (out_max_iter != -1 && iter == out_max_iter) || (swap_cnt >= 10 && fabs(diff[0] - 2.0) > eps))
            break;
    }
    if (stats) {
        stats[0] = iter + 1;
        stats[1] = (double) local_iter;
        stats[2] = diff[0];
        stats[3] = oracle_objective(n, f_val, alpha, y);
    }
    *rho_out = solver_kind == 0 ? rho_c(n, f_val, y, alpha, Cp, Cn)
                                : rho_nu(n, f_val, y, alpha, Cp, Cn, solver_kind == 2);
    free(sd); free(diag); free(ws); free(order); free(ind); free(srt); free(alpha_diff); free(rows);
}

/* sum_kernel_values (kernelmatrix_kernel.cpp:110-147): dec[r*nb + k] for every class pair */
void oracle_sum_kernel_values(const double *coef, int total_sv, const int *sv_start, const int *sv_count,
                              const double *rho, const float *k_mat, double *dec, int n_classes, int m) {
    const int nb = n_classes * (n_classes - 1) / 2;
#pragma omp parallel for schedule(guided)
    for (int r = 0; r < m; ++r) {
        int k = 0;
        const float *kv = k_mat + (size_t) r * total_sv;
        for (int i = 0; i < n_classes; ++i)
            for (int j = i + 1; j < n_classes; ++j) {
                const double *c1 = coef + (size_t) (j - 1) * total_sv, *c2 = coef + (size_t) i * total_sv;
                double s = 0;
                for (int l = 0; l < sv_count[i]; ++l) s += c1[sv_start[i] + l] * kv[sv_start[i] + l];
                for (int l = 0; l < sv_count[j]; ++l) s += c2[sv_start[j] + l] * kv[sv_start[j] + l];
                dec[(size_t) r * nb + k] = s - rho[k];
                k++;
            }
    }
}

/* SvmModel::predict_dec_values (svmmodel.cpp:74-117) for one batch holding all m rows */
void oracle_predict_dec(int n_sv, int n_features, const float *val, const int *row_ptr, const int *col, int kernel,
                        int degree, float gamma, float coef0, const double *coef, const int *sv_count, const double *rho,
                        int n_classes, int m, const float *tval, const int *trow_ptr, const int *tcol, double *dec) {
    float *K = malloc(sizeof(float) * (size_t) m * n_sv);
    int *sv_start = malloc(sizeof(int) * n_classes);
    sv_start[0] = 0;
    for (int i = 1; i < n_classes; ++i) sv_start[i] = sv_start[i - 1] + sv_count[i - 1];
    oracle_kernel_rows_ins(n_sv, n_features, val, row_ptr, col, kernel, degree, gamma, coef0, m, tval, trow_ptr, tcol,
                           K);
    oracle_sum_kernel_values(coef, n_sv, sv_start, sv_count, rho, K, dec, n_classes, m);
    free(K);
    free(sv_start);
}

/* SVC::predict_label voting (svc.cpp:265-289): out[r] = winning class INDEX */
void oracle_vote(const double *dec, int m, int n_classes, int *out) {
    const int nb = n_classes * (n_classes - 1) / 2;
    int *votes = malloc(sizeof(int) * n_classes);
    for (int r = 0; r < m; ++r) {
        memset(votes, 0, sizeof(int) * n_classes);
        int k = 0;
        for (int i = 0; i < n_classes; ++i)
            for (int j = i + 1; j < n_classes; ++j) {
                if (dec[(size_t) r * nb + k] > 0) votes[i]++; else votes[j]++;
                k++;
            }
        int best = 0;
        for (int i = 1; i < n_classes; ++i) if (votes[i] > votes[best]) best = i;
        out[r] = best;
    }
    free(votes);
}
