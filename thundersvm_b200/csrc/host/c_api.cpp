// The reference's exported C symbols, unchanged in name and argument order, so that its Python
// package (python/thundersvm/thundersvm.py loads the library with ctypes) and its Matlab / command
// string front ends keep working against this library:
//   scikit-style API   src/thundersvm/thundersvm-scikit.cpp:15-400
//   command-line API   src/thundersvm/svm_interface_api.cpp:94-205
#include <thundersvm/model/svc.h>
#include <thundersvm/model/nusvc.h>
#include <thundersvm/model/svr.h>
#include <thundersvm/model/nusvr.h>
#include <thundersvm/model/oneclass_svc.h>
#include <thundersvm/cmdparser.h>
#include <thundersvm/util/metric.h>
#include <thundersvm/svm_interface_api.h>
#include <cuda_runtime.h>
#include <cstring>
#include <fstream>
#include <memory>
#include <omp.h>

namespace {
SvmModel *new_model(int svm_type) {
    switch (svm_type) {
        case SvmParam::C_SVC: return new SVC();
        case SvmParam::NU_SVC: return new NuSVC();
        case SvmParam::ONE_CLASS: return new OneClassSVC();
        case SvmParam::EPSILON_SVR: return new SVR();
        case SvmParam::NU_SVR: return new NuSVR();
    }
    return nullptr;
}

bool nu_feasible(DataSet &ds, double nu) {
    ds.group_classes();
    for (size_t i = 0; i < ds.n_classes(); ++i)
        for (size_t j = i + 1; j < ds.n_classes(); ++j) {
            const int n1 = ds.count()[i], n2 = ds.count()[j];
            if (nu * (n1 + n2) / 2 > std::min(n1, n2)) return false;
        }
    return true;
}

void train_common(DataSet &train, int svm_type, int kernel_type, int degree, float gamma, float coef0, float cost,
                  float nu, float epsilon, float tol, int probability, int weight_size, int *weight_label,
                  float *weight, int verbose, int max_iter, int n_cores, int max_mem_size, int gpu_id, int *n_features,
                  int *n_classes, int *succeed, SvmModel *model) {
    cudaSetDevice(gpu_id);
    succeed[0] = 1;
    thundersvm::set_verbose(verbose != 0);
    if (n_cores > 0) omp_set_num_threads(n_cores);
    else if (n_cores != -1) LOG(ERROR) << "n_jobs must be positive or -1";
    model->set_max_iter(max_iter);
    if (svm_type == SvmParam::NU_SVC && !nu_feasible(train, nu)) {
        printf("specified nu is infeasible\n");
        succeed[0] = -1;
    }
    SvmParam p;
    p.svm_type = static_cast<SvmParam::SVM_TYPE>(svm_type);
    p.kernel_type = static_cast<SvmParam::KERNEL_TYPE>(kernel_type);
    p.degree = degree;
    p.gamma = gamma;
    p.coef0 = coef0;
    p.C = cost;
    p.nu = nu;
    p.p = epsilon;
    p.epsilon = tol;
    p.probability = probability;
    if (max_mem_size != -1) p.max_mem_size = static_cast<size_t>(std::max(max_mem_size, 0)) << 20;
    if (weight_size != 0) {
        p.nr_weight = weight_size;
        p.weight = (float_type *) malloc(weight_size * sizeof(float_type));
        p.weight_label = (int *) malloc(weight_size * sizeof(int));
        for (int i = 0; i < weight_size; ++i) { p.weight[i] = weight[i]; p.weight_label[i] = weight_label[i]; }
    }
    model->train(train, p);
    LOG(INFO) << "training finished";
    n_features[0] = (int) train.n_features();
    n_classes[0] = model->get_n_classes();
}

void copy_out(const vector<float_type> &src, float *dst) {
    for (size_t i = 0; i < src.size(); ++i) dst[i] = (float) src[i];
}

DataSet g_python_dataset;        // filled by load_from_python_interface, consumed by the *_after_parse calls
}  // namespace

extern "C" {

SvmModel *model_new(int svm_type) { return new_model(svm_type); }
void model_free(SvmModel *model) { delete model; }

void init_model_param(char *kernel_type, int *degree, float *gamma, float *coef0, int *probability, SvmModel *model) {
    model->get_param(kernel_type, degree, gamma, coef0, probability);
}

void sparse_model_scikit(int row_size, float *val, int *row_ptr, int *col_ptr, float *label, int svm_type,
                         int kernel_type, int degree, float gamma, float coef0, float cost, float nu, float epsilon,
                         float tol, int probability, int weight_size, int *weight_label, float *weight, int verbose,
                         int max_iter, int n_cores, int max_mem_size, int gpu_id, int *n_features, int *n_classes,
                         int *succeed, SvmModel *model) {
    DataSet train;
    thundersvm::set_verbose(verbose != 0);
    train.load_from_sparse(row_size, val, row_ptr, col_ptr, label);
    train_common(train, svm_type, kernel_type, degree, gamma, coef0, cost, nu, epsilon, tol, probability, weight_size,
                 weight_label, weight, verbose, max_iter, n_cores, max_mem_size, gpu_id, n_features, n_classes, succeed,
                 model);
}

void dense_model_scikit(int row_size, int features, float *data, float *label, int svm_type, int kernel_type,
                        int degree, float gamma, float coef0, float cost, float nu, float epsilon, float tol,
                        int probability, int weight_size, int *weight_label, float *weight, int verbose, int max_iter,
                        int n_cores, int max_mem_size, int gpu_id, int *n_features, int *n_classes, int *succeed,
                        SvmModel *model) {
    DataSet train;
    thundersvm::set_verbose(verbose != 0);
    train.load_from_dense(row_size, features, data, label);
    train_common(train, svm_type, kernel_type, degree, gamma, coef0, cost, nu, epsilon, tol, probability, weight_size,
                 weight_label, weight, verbose, max_iter, n_cores, max_mem_size, gpu_id, n_features, n_classes, succeed,
                 model);
}

int sparse_predict(int row_size, float *val, int *row_ptr, int *col_ptr, SvmModel *model, float *predict_label,
                   int verbose) {
    thundersvm::set_verbose(verbose != 0);
    DataSet ds;
    ds.load_from_sparse(row_size, val, row_ptr, col_ptr, nullptr);
    copy_out(model->predict(ds.instances(), -1), predict_label);
    return 0;
}

int dense_predict(int row_size, int features, float *data, SvmModel *model, float *predict_label, int verbose) {
    thundersvm::set_verbose(verbose != 0);
    DataSet ds;
    ds.load_from_dense(row_size, features, data, nullptr);
    copy_out(model->predict(ds.instances(), -1), predict_label);
    return 0;
}

void sparse_decision(int row_size, float *val, int *row_ptr, int *col_ptr, SvmModel *model, int value_size,
                     float *dec_value) {
    DataSet ds;
    ds.load_from_sparse(row_size, val, row_ptr, col_ptr, nullptr);
    model->predict(ds.instances(), -1);
    const SyncArray<float_type> &d = model->get_dec_value();
    for (size_t i = 0; i < d.size() && (int) i < value_size; ++i) dec_value[i] = (float) d.host_data()[i];
}

void dense_decision(int row_size, int features, float *data, SvmModel *model, int value_size, float *dec_value) {
    DataSet ds;
    ds.load_from_dense(row_size, features, data, nullptr);
    model->predict(ds.instances(), -1);
    const SyncArray<float_type> &d = model->get_dec_value();
    for (size_t i = 0; i < d.size() && (int) i < value_size; ++i) dec_value[i] = (float) d.host_data()[i];
}

int n_sv(SvmModel *model) { return model->total_sv(); }
void set_iter(SvmModel *model, int iter) { model->set_max_iter(iter); }
void set_memory_size(SvmModel *model, int m_size) { model->set_max_memory_size(m_size); }

void get_sv(int *row, int *col, float *data, int *data_size, int *sv_indices, SvmModel *model) {
    const DataSet::node2d &svs = model->svs();
    int p = 0;
    row[0] = 0;
    for (size_t i = 0; i < svs.size(); ++i) {
        for (auto &nd : svs[i]) { data[p] = nd.value; col[p] = nd.index; ++p; }
        row[i + 1] = p;
    }
    data_size[0] = p;
    const vector<int> &ids = model->get_sv_ind();
    for (size_t i = 0; i < ids.size(); ++i) sv_indices[i] = ids[i];
}

void get_support_classes(int *n_support, int n_class, SvmModel *model) {
    const SyncArray<int> &c = model->get_n_sv();
    for (int i = 0; i < n_class && i < (int) c.size(); ++i) n_support[i] = c.host_data()[i];
}

void get_coef(float *dual_coef, int n_class, int n_sv_, SvmModel *model) {
    const SyncArray<float_type> &c = model->get_coef();
    for (size_t i = 0; i < c.size() && i < (size_t) (n_class - 1) * n_sv_; ++i) dual_coef[i] = (float) c.host_data()[i];
}

void get_linear_coef(float *linear_coef, int n_binary_model, int n_feature, SvmModel *model) {
    const SyncArray<float_type> &c = model->get_linear_coef();
    for (size_t i = 0; i < c.size() && i < (size_t) n_binary_model * n_feature; ++i) linear_coef[i] = (float) c.host_data()[i];
}

void get_rho(float *rho_, int rho_size, SvmModel *model) {
    const SyncArray<float_type> &r = model->get_rho();
    for (int i = 0; i < rho_size && i < (int) r.size(); ++i) rho_[i] = (float) r.host_data()[i];
}

void get_pro(SvmModel *model, float *prob) {
    const vector<float> &p = model->get_prob_predict();
    for (size_t i = 0; i < p.size(); ++i) prob[i] = p[i];
}

void get_n_binary_models(SvmModel *model, int *n_model) { n_model[0] = model->get_n_binary_models(); }
void get_n_classes(SvmModel *model, int *n_classes) { n_classes[0] = model->get_n_classes(); }
void get_sv_max_index(SvmModel *model, int *n_feature) { n_feature[0] = model->get_sv_max_index(); }

void save_to_file_scikit(SvmModel *model, char *path) { model->save_to_file(path); }
void load_from_file_scikit(SvmModel *model, char *path) { model->load_from_file(path); }

// malloc'd, NOT NUL-terminated copy of the model text; release with free_string
char *save_to_string_scikit(SvmModel *model) {
    const string s = model->save_to_string();
    char *buf = (char *) malloc(s.length());
    memcpy(buf, s.c_str(), s.length());
    return buf;
}
void free_string(char *s) { free(s); }
void load_from_string_scikit(SvmModel *model, char *mstring) { model->load_from_string(string(mstring)); }

// ---- command-line style API ------------------------------------------------------------------------
static void run_train(CMDParser &parser, DataSet &train) {
    std::unique_ptr<SvmModel> model(new_model(parser.param_cmd.svm_type));
    if (parser.param_cmd.svm_type == SvmParam::NU_SVC && !nu_feasible(train, parser.param_cmd.nu)) {
        printf("specified nu is infeasible\n");
        return;
    }
    if (parser.param_cmd.kernel_type != SvmParam::LINEAR) {
        if (!parser.gamma_set) {
            parser.param_cmd.gamma = 1.f / train.n_features();
            LOG(WARNING) << "using default gamma=" << parser.param_cmd.gamma;
        } else LOG(INFO) << "gamma = " << parser.param_cmd.gamma;
    }
    cudaSetDevice(parser.gpu_id);
    if (parser.do_cross_validation) {
        vector<float_type> y = model->cross_validation(train, parser.param_cmd, parser.nr_fold);
        std::unique_ptr<Metric> metric;
        if (parser.param_cmd.svm_type <= SvmParam::NU_SVC) metric.reset(new Accuracy());
        else if (parser.param_cmd.svm_type >= SvmParam::EPSILON_SVR) metric.reset(new MSE());
        if (metric) std::cout << "Cross " << metric->name() << " = " << metric->score(y, train.y()) << std::endl;
    } else {
        model->train(train, parser.param_cmd);
        LOG(INFO) << "training finished";
        model->save_to_file(parser.model_file_name);
    }
}

static void run_predict(const string &model_file, const string &out_file, DataSet &test, size_t max_mem, int gpu_id) {
    std::ifstream f(model_file);
    if (!f.is_open()) { LOG(INFO) << "file " << model_file << " not found"; exit(1); }
    string key, type;
    f >> key >> type;
    CHECK_EQ(key, "svm_type");
    int st = 0;
    for (int i = 0; i < 5; ++i) if (type == SvmParam::svm_type_name[i]) st = i;
    std::unique_ptr<SvmModel> model(new_model(st));
    std::unique_ptr<Metric> metric;
    if (st <= SvmParam::NU_SVC) metric.reset(new Accuracy());
    else if (st >= SvmParam::EPSILON_SVR) metric.reset(new MSE());
    cudaSetDevice(gpu_id);
    model->set_max_memory_size_Byte(max_mem);
    model->load_from_file(model_file);
    vector<float_type> y = model->predict(test.instances(), -1);
    std::ofstream out(out_file);
    if (model->is_prob()) {
        const vector<int> &lab = model->get_label();
        const vector<float> &pp = model->get_prob_predict();
        out << "labels ";
        for (int l : lab) out << l << " ";
        out << std::endl;
        for (size_t i = 0; i < y.size(); ++i) {
            out << y[i] << " ";
            for (size_t j = 0; j < lab.size(); ++j) out << pp[lab.size() * i + j] << " ";
            out << std::endl;
        }
    } else
        for (float_type v : y) out << v << std::endl;
    if (metric && test.y().size() == y.size()) LOG(INFO) << metric->name() << " = " << metric->score(y, test.y());
}

void thundersvm_train(int argc, char **argv) {
    CMDParser parser;
    parser.parse_command_line(argc, argv);
    DataSet train;
    train.load_from_file(parser.svmtrain_input_file_name);
    run_train(parser, train);
}

void thundersvm_train_after_parse(char **option, int len, char *file_name) {
    CMDParser parser;
    parser.parse_python(len, option);
    parser.model_file_name = file_name;
    run_train(parser, g_python_dataset);
}

void thundersvm_predict(int argc, char **argv) {
    CMDParser parser;
    parser.parse_command_line(argc, argv);
    DataSet test;
    test.load_from_file(parser.svmpredict_input_file);
    run_predict(parser.svmpredict_model_file_name, parser.svmpredict_output_file, test, parser.param_cmd.max_mem_size,
                parser.gpu_id);
}

void thundersvm_predict_after_parse(char *model_file_name, char *output_file_name, char **option, int len) {
    CMDParser parser;
    parser.parse_python(len, option);
    run_predict(model_file_name, output_file_name, g_python_dataset, parser.param_cmd.max_mem_size, parser.gpu_id);
}

void load_from_python_interface(float *y, char **x, int len) { g_python_dataset.load_from_python(y, x, len); }

}  // extern "C"
