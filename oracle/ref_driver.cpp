// TEST INFRASTRUCTURE ONLY - a C-callable driver around the *reference's own* CPU
// objects (compiled unmodified from the reference source tree by oracle/Makefile
// into oracle/_ref/libthundersvm_ref.so). It is loaded by the tests, by the smoke
// check and by the benchmark's CPU-baseline / reference arm as the checker and the
// timed CPU baseline. The product library never links or calls it.
//
// The driver feeds seeded arrays straight into the reference classes:
//   DataSet::load_from_dense / load_from_sparse  (src/thundersvm/dataset.cpp:124-172)
//   KernelMatrix::{get_rows x2, diag}            (src/thundersvm/kernelmatrix.cpp:251-316)
//   CSMOSolver / NuSMOSolver ::solve             (src/thundersvm/solver/csmosolver.cpp:10-121)
//   SvmModel::{train, predict, predict_dec_values, cross_validation, save_to_string}
// Column indices arrive 0-based and are shifted to the 1-based LibSVM convention
// exactly as load_from_sparse does (dataset.cpp:136-137).
#include <thundersvm/dataset.h>
#include <thundersvm/kernelmatrix.h>
#include <thundersvm/solver/csmosolver.h>
#include <thundersvm/solver/nusmosolver.h>
#include <thundersvm/model/svc.h>
#include <thundersvm/model/nusvc.h>
#include <thundersvm/model/svr.h>
#include <thundersvm/model/nusvr.h>
#include <thundersvm/model/oneclass_svc.h>
#include <chrono>
#include <cstring>
#include <omp.h>

namespace {
    double now_s() {
        return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
    }

    // dense != NULL: n x d row-major, explicit zeros kept (dataset.cpp:150-172).
    // else CSR with 0-based columns (dataset.cpp:124-148).
    void fill_dataset(DataSet &ds, int n, int d, const float *dense, const float *val, const int *row_ptr,
                      const int *col, const float *label) {
        if (dense) ds.load_from_dense(n, d, const_cast<float *>(dense), const_cast<float *>(label));
        else
            ds.load_from_sparse(n, const_cast<float *>(val), const_cast<int *>(row_ptr), const_cast<int *>(col),
                                const_cast<float *>(label));
    }

    SvmParam make_param(int svm_type, int ktype, int degree, double gamma, double coef0, double C, double nu,
                        double p, double eps, int probability) {
        SvmParam prm;
        prm.svm_type = static_cast<SvmParam::SVM_TYPE>(svm_type);
        prm.kernel_type = static_cast<SvmParam::KERNEL_TYPE>(ktype);
        prm.degree = degree;
        prm.gamma = gamma;
        prm.coef0 = coef0;
        prm.C = C;
        prm.nu = nu;
        prm.p = p;
        prm.epsilon = eps;
        prm.probability = probability;
        prm.max_mem_size = static_cast<size_t>(1) << 40;  // never the limiting factor here
        return prm;
    }

    struct RefModel {
        SvmModel *model = nullptr;
        int svm_type = 0;
    };
}

extern "C" {

void ref_set_quiet(int quiet) {
    el::Loggers::reconfigureAllLoggers(el::ConfigurationType::Enabled, quiet ? "false" : "true");
}

void ref_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

int ref_max_threads() { return omp_get_max_threads(); }

// Kernel rows by index: out[q x n] row-major. Returns seconds spent in `reps`
// repetitions of get_rows (construction excluded).
double ref_kernel_rows_idx(int n, int d, const float *dense, const float *val, const int *row_ptr, const int *col,
                           int ktype, int degree, double gamma, double coef0, const int *idx, int q, float *out,
                           float *diag_out, int reps) {
    DataSet ds;
    fill_dataset(ds, n, d, dense, val, row_ptr, col, nullptr);
    SvmParam prm = make_param(0, ktype, degree, gamma, coef0, 1, 0.5, 0.1, 1e-3, 0);
    KernelMatrix km(ds.instances(), prm);
    SyncArray<int> ids(q);
    ids.copy_from(idx, q);
    SyncArray<kernel_type> rows((size_t) q * n);
    double t0 = now_s();
    for (int r = 0; r < (reps < 1 ? 1 : reps); ++r) km.get_rows(ids, rows);
    double t1 = now_s();
    if (out) memcpy(out, rows.host_data(), sizeof(float) * (size_t) q * n);
    if (diag_out) memcpy(diag_out, km.diag().host_data(), sizeof(float) * n);
    return t1 - t0;
}

// Kernel values of m new instances against the n stored ones: out[m x n] row-major.
double ref_kernel_rows_ins(int n, int d, const float *dense, const float *val, const int *row_ptr, const int *col,
                           int m, int d2, const float *dense2, const float *val2, const int *row_ptr2, const int *col2,
                           int ktype, int degree, double gamma, double coef0, float *out) {
    DataSet ds, ts;
    fill_dataset(ds, n, d, dense, val, row_ptr, col, nullptr);
    fill_dataset(ts, m, d2, dense2, val2, row_ptr2, col2, nullptr);
    SvmParam prm = make_param(0, ktype, degree, gamma, coef0, 1, 0.5, 0.1, 1e-3, 0);
    KernelMatrix km(ds.instances(), prm);
    SyncArray<kernel_type> rows((size_t) m * n);
    double t0 = now_s();
    km.get_rows(ts.instances(), rows);
    double t1 = now_s();
    memcpy(out, rows.host_data(), sizeof(float) * (size_t) m * n);
    return t1 - t0;
}

// One call of CSMOSolver::solve (solver_kind 0) or NuSMOSolver::solve
// (1 = nu-SVC scaling, 2 = nu-SVR, no scaling). alpha and f_val are in/out.
// Returns seconds spent inside solve().
double ref_smo_solve(int n, int d, const float *dense, const float *val, const int *row_ptr, const int *col,
                     int ktype, int degree, double gamma, double coef0, int solver_kind, const int *y,
                     double *alpha, double *f_val, double eps, double Cp, double Cn, int ws_size, int max_iter,
                     double *rho_out) {
    DataSet ds;
    fill_dataset(ds, n, d, dense, val, row_ptr, col, nullptr);
    SvmParam prm = make_param(0, ktype, degree, gamma, coef0, 1, 0.5, 0.1, eps, 0);
    KernelMatrix km(ds.instances(), prm);
    SyncArray<int> ya(n);
    ya.copy_from(y, n);
    SyncArray<float_type> a(n), f(n);
    a.copy_from(alpha, n);
    f.copy_from(f_val, n);
    float_type rho = 0;
    double t0 = now_s();
    if (solver_kind == 0) {
        CSMOSolver s;
        s.solve(km, ya, a, rho, f, eps, Cp, Cn, ws_size, max_iter);
    } else {
        NuSMOSolver s(solver_kind == 2);
        s.solve(km, ya, a, rho, f, eps, Cp, Cn, ws_size, max_iter);
    }
    double t1 = now_s();
    memcpy(alpha, a.host_data(), sizeof(double) * n);
    memcpy(f_val, f.host_data(), sizeof(double) * n);
    *rho_out = rho;
    return t1 - t0;
}

// ---- model-level API (train / predict / introspection) -------------------------
void *ref_model_train(int svm_type, int n, int d, const float *dense, const float *val, const int *row_ptr,
                      const int *col, const float *label, int ktype, int degree, double gamma, double coef0,
                      double C, double nu, double p, double eps, int probability, int max_iter,
                      double *train_seconds) {
    DataSet ds;
    fill_dataset(ds, n, d, dense, val, row_ptr, col, label);
    SvmParam prm = make_param(svm_type, ktype, degree, gamma, coef0, C, nu, p, eps, probability);
    RefModel *rm = new RefModel;
    rm->svm_type = svm_type;
    switch (svm_type) {
        case SvmParam::C_SVC: rm->model = new SVC(); break;
        case SvmParam::NU_SVC: rm->model = new NuSVC(); break;
        case SvmParam::ONE_CLASS: rm->model = new OneClassSVC(); break;
        case SvmParam::EPSILON_SVR: rm->model = new SVR(); break;
        default: rm->model = new NuSVR(); break;
    }
    rm->model->set_max_iter(max_iter);
    // region timed by the reference CLI: src/thundersvm/thundersvm-train.cpp:89-94
    double t0 = now_s();
    rm->model->train(ds, prm);
    double t1 = now_s();
    if (train_seconds) *train_seconds = t1 - t0;
    return rm;
}

void ref_model_free(void *h) {
    RefModel *rm = static_cast<RefModel *>(h);
    if (!rm) return;
    delete rm->model;
    delete rm;
}

// info[0]=n_classes, [1]=n_binary_models, [2]=total_sv
void ref_model_info(void *h, int *info) {
    RefModel *rm = static_cast<RefModel *>(h);
    info[0] = rm->model->get_n_classes();
    info[1] = rm->model->get_n_binary_models();
    info[2] = rm->model->total_sv();
}

void ref_model_get(void *h, double *rho, double *coef, int *n_sv, int *sv_ind, int *labels) {
    RefModel *rm = static_cast<RefModel *>(h);
    SvmModel *m = rm->model;
    if (rho) memcpy(rho, m->get_rho().host_data(), sizeof(double) * m->get_rho().size());
    if (coef) memcpy(coef, m->get_coef().host_data(), sizeof(double) * m->get_coef().size());
    if (n_sv) memcpy(n_sv, m->get_n_sv().host_data(), sizeof(int) * m->get_n_sv().size());
    if (sv_ind) memcpy(sv_ind, m->get_sv_ind().data(), sizeof(int) * m->get_sv_ind().size());
    if (labels) memcpy(labels, m->get_label().data(), sizeof(int) * m->get_label().size());
}

int ref_model_coef_size(void *h) { return (int) static_cast<RefModel *>(h)->model->get_coef().size(); }

// predict: labels_out[m] (class label / regression value / +-1); dec_out may be
// NULL, else m x n_binary_models decision values (svmmodel.cpp:74-117).
double ref_model_predict(void *h, int m, int d, const float *dense, const float *val, const int *row_ptr,
                         const int *col, double *labels_out, double *dec_out) {
    RefModel *rm = static_cast<RefModel *>(h);
    DataSet ts;
    fill_dataset(ts, m, d, dense, val, row_ptr, col, nullptr);
    double t0 = now_s();
    vector<float_type> yp = rm->model->predict(ts.instances(), -1);
    double t1 = now_s();
    if (labels_out) memcpy(labels_out, yp.data(), sizeof(double) * yp.size());
    if (dec_out) {
        int nb = rm->model->get_n_binary_models();
        SyncArray<float_type> dec((size_t) m * nb);
        rm->model->predict_dec_values(ts.instances(), dec, -1);
        memcpy(dec_out, dec.host_data(), sizeof(double) * (size_t) m * nb);
    }
    return t1 - t0;
}

// 5-fold style cross validation (svmmodel.cpp:31-71); out[n] predictions.
void ref_cross_validation(int svm_type, int n, int d, const float *dense, const float *val, const int *row_ptr,
                          const int *col, const float *label, int ktype, int degree, double gamma,
                          double coef0, double C, double nu, double p, double eps, int n_fold, double *out) {
    DataSet ds;
    fill_dataset(ds, n, d, dense, val, row_ptr, col, label);
    SvmParam prm = make_param(svm_type, ktype, degree, gamma, coef0, C, nu, p, eps, 0);
    SvmModel *model;
    switch (svm_type) {
        case SvmParam::C_SVC: model = new SVC(); break;
        case SvmParam::NU_SVC: model = new NuSVC(); break;
        case SvmParam::ONE_CLASS: model = new OneClassSVC(); break;
        case SvmParam::EPSILON_SVR: model = new SVR(); break;
        default: model = new NuSVR(); break;
    }
    vector<float_type> yp = model->cross_validation(ds, prm, n_fold);
    memcpy(out, yp.data(), sizeof(double) * yp.size());
    delete model;
}

// Model text in the LibSVM-compatible format (svmmodel.cpp:193-264). Returns the
// length; copies at most cap bytes into buf.
long ref_model_save_to_string(void *h, char *buf, long cap) {
    RefModel *rm = static_cast<RefModel *>(h);
    string s = rm->model->save_to_string();
    long n = (long) s.size();
    if (buf && cap > 0) memcpy(buf, s.data(), n < cap ? n : cap);
    return n;
}

}  // extern "C"
