// The model layer: SvmModel and its five concrete models. Problem set-up, support-vector
// extraction, voting / probabilities, cross validation and the LibSVM-compatible model text follow
// the reference (src/thundersvm/model/{svmmodel,svc,nusvc,svr,nusvr,oneclass_svc}.cpp); every
// numerical step goes through KernelMatrix / CSMOSolver / NuSMOSolver or the C ABI directly.
#include <atomic>
#include <exception>
#include <mutex>
#include <thread>
#include <thundersvm/model/svmmodel.h>
#include <thundersvm/model/svc.h>
#include <thundersvm/model/nusvc.h>
#include <thundersvm/model/svr.h>
#include <thundersvm/model/nusvr.h>
#include <thundersvm/model/oneclass_svc.h>
#include <thundersvm/solver/csmosolver.h>
#include <thundersvm/solver/nusmosolver.h>
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <memory>
#include <cuda_runtime.h>
#include "../../../include/thundersvm_b200.h"

namespace {
void b200_check(tsvm_status s) {
    if (s == TSVM_OK) return;
    if (s == TSVM_ERR_OOM) throw std::bad_alloc();
    LOG(FATAL) << "thundersvm_b200: " << tsvm_last_error();
}

// Splits every class into n_fold contiguous slices of its grouped order; fold k tests slice k (the
// last fold takes the remainder), svmmodel.cpp:40-60 / svc.cpp:436-459.
void fold_split(const DataSet &ds, int n_fold, int k, DataSet::node2d &x_train, vector<float_type> &y_train,
                DataSet::node2d &x_test, vector<float_type> &y_test, vector<int> &test_idx) {
    for (size_t c = 0; c < ds.n_classes(); ++c) {
        const vector<int> ids = ds.original_index((int) c);
        const int per = ds.count()[c] / n_fold;
        const int b = per * k;
        const int e = (k == n_fold - 1) ? (int) ids.size() : std::min<int>(b + per, (int) ids.size());
        for (int t = 0; t < (int) ids.size(); ++t) {
            const int j = ids[t];
            if (t >= b && t < e) { x_test.push_back(ds.instances()[j]); y_test.push_back(ds.y()[j]); test_idx.push_back(j); }
            else { x_train.push_back(ds.instances()[j]); y_train.push_back(ds.y()[j]); }
        }
    }
}
}  // namespace

// ------------------------------------------------------------------------------------------------
// SvmModel
// ------------------------------------------------------------------------------------------------
void SvmModel::model_setup(const DataSet &dataset, SvmParam &param) {
    n_binary_models = (size_t) n_classes * (n_classes - 1) / 2;
    rho.resize(n_binary_models);
    n_sv.resize(n_classes);
    sv.clear();
    sv_indices.clear();
    invalidate_sv_matrix();
    this->param = param;
}

const KernelMatrix &SvmModel::sv_matrix() const {
    if (!sv_kmat_ || sv_kmat_->n_instances() != sv.size()) sv_kmat_.reset(new KernelMatrix(sv, param));
    return *sv_kmat_;
}

int SvmModel::get_working_set_size(int n_instances, int n_features) {
    const int ws = tsvm_working_set_size(n_instances, n_features, param.max_mem_size, thundersvm::total_memory_size());
    if (ws < 0) throw std::bad_alloc();          // the budget is already exceeded (svmmodel.cpp:440-442)
    LOG(INFO) << "working set size = " << ws;
    return ws;
}

vector<float_type> SvmModel::cross_validation(DataSet dataset, SvmParam param, int n_fold) {
    dataset.group_classes(this->param.svm_type == SvmParam::C_SVC);
    vector<float_type> y_all(dataset.n_instances());
    for (int k = 0; k < n_fold; ++k) {
        LOG(INFO) << n_fold << " fold cross-validation (" << k + 1 << "/" << n_fold << ")";
        DataSet::node2d x_train, x_test;
        vector<float_type> y_train, y_test;
        vector<int> test_idx;
        fold_split(dataset, n_fold, k, x_train, y_train, x_test, y_test, test_idx);
        DataSet train_set(x_train, (int) dataset.n_features(), y_train);
        this->train(train_set, param);
        vector<float_type> y_pred = this->predict(x_test, 1000);
        CHECK_EQ(y_pred.size(), test_idx.size());
        for (size_t i = 0; i < y_pred.size(); ++i) y_all[test_idx[i]] = y_pred[i];
    }
    return y_all;
}

void SvmModel::predict_dec_values(const DataSet::node2d &instances, SyncArray<float_type> &dec_values,
                                  int batch_size) const {
    const size_t m = instances.size();
    if (m == 0) return;
    CHECK_GE(dec_values.size(), m * n_binary_models) << "dec_values is too small";
    if (sv.empty()) {                       // no support vector: the decision value is -rho
        float_type *d = dec_values.host_data();
        for (size_t r = 0; r < m; ++r)
            for (size_t k = 0; k < n_binary_models; ++k) d[r * n_binary_models + k] = -rho.host_data()[k];
        return;
    }
    const KernelMatrix &k_mat = sv_matrix();
    // test batch as CSR on the device
    size_t nnz = 0;
    for (auto &r : instances) nnz += r.size();
    SyncArray<kernel_type> tval(std::max<size_t>(nnz, 1));
    SyncArray<int> tcol(std::max<size_t>(nnz, 1)), trp(m + 1);
    {
        kernel_type *v = tval.host_data();
        int *c = tcol.host_data(), *rp = trp.host_data();
        size_t p = 0;
        rp[0] = 0;
        for (size_t r = 0; r < m; ++r) {
            for (auto &nd : instances[r]) { v[p] = nd.value; c[p] = nd.index; ++p; }
            rp[r + 1] = (int) p;
        }
    }
    size_t budget = 0;                      // 0 = library default; a positive batch size bounds the K buffer
    if (batch_size > 0) budget = (size_t) batch_size * (((size_t) sv.size() + 3) & ~3ul) * sizeof(kernel_type);
    b200_check(tsvm_predict_dec(k_mat.handle(), coef.device_data(), n_sv.host_data(), rho.device_data(), n_classes,
                                (int) m, nullptr, 0, 0, tval.device_data(), trp.device_data(), tcol.device_data(),
                                (long long) nnz, dec_values.device_data(), budget, nullptr));
}

// Test batch as CSR arrays on the device.
struct DeviceBatch {
    SyncArray<kernel_type> val;
    SyncArray<int> col, row_ptr;
    size_t nnz = 0;
    explicit DeviceBatch(const DataSet::node2d &instances) {
        for (auto &r : instances) nnz += r.size();
        val.resize(std::max<size_t>(nnz, 1));
        col.resize(std::max<size_t>(nnz, 1));
        row_ptr.resize(instances.size() + 1);
        kernel_type *v = val.host_data();
        int *c = col.host_data(), *rp = row_ptr.host_data();
        size_t p = 0;
        rp[0] = 0;
        for (size_t r = 0; r < instances.size(); ++r) {
            for (auto &nd : instances[r]) { v[p] = nd.value; c[p] = nd.index; ++p; }
            rp[r + 1] = (int) p;
        }
    }
};

void SvmModel::predict_dec_values_instant(const DataSet::node2d &instances, SyncArray<float_type> &predict_instant,
                                          int batch_size) const {
    // svmmodel.cpp:119-154 + sum_kernel_values_instant: only the winning class index of every row leaves the
    // device; the decision values live in a slab-sized scratch inside tsvm_predict_labels
    const size_t m = instances.size();
    if (m == 0) return;
    float_type *out = predict_instant.host_data();
    if (sv.empty()) {                       // every decision value is -rho: the vote is the same for all rows
        for (size_t r = 0; r < m; ++r) {
            vector<int> votes(n_classes, 0);
            size_t k = 0;
            for (int i = 0; i < n_classes; ++i)
                for (int j = i + 1; j < n_classes; ++j, ++k) votes[-rho.host_data()[k] > 0 ? i : j]++;
            out[r] = (float_type) (std::max_element(votes.begin(), votes.end()) - votes.begin());
        }
        return;
    }
    const KernelMatrix &k_mat = sv_matrix();
    DeviceBatch batch(instances);
    size_t budget = 0;
    if (batch_size > 0) budget = (size_t) batch_size * (((size_t) sv.size() + 3) & ~3ul) * sizeof(kernel_type);
    SyncArray<int> winner(m);
    b200_check(tsvm_predict_labels(k_mat.handle(), coef.device_data(), n_sv.host_data(), rho.device_data(), n_classes,
                                   (int) m, nullptr, 0, 0, batch.val.device_data(), batch.row_ptr.device_data(),
                                   batch.col.device_data(), (long long) batch.nnz, winner.device_data(), budget,
                                   nullptr));
    const int *w = winner.host_data();
    for (size_t r = 0; r < m; ++r) out[r] = w[r];
}

vector<float_type> SvmModel::predict(const DataSet::node2d &instances, int batch_size = -1) {
    dec_values.resize(instances.size() * n_binary_models);
    predict_dec_values(instances, dec_values, batch_size);
    const float_type *d = dec_values.host_data();
    return vector<float_type>(d, d + dec_values.size());
}

vector<float_type> SvmModel::predict_instant(const DataSet::node2d &instances, int batch_size) {
    SyncArray<float_type> idx(instances.size());
    predict_dec_values_instant(instances, idx, batch_size);
    vector<float_type> out(instances.size());
    for (size_t i = 0; i < out.size(); ++i) out[i] = (float) label[(int) idx.host_data()[i]];
    return out;
}

void SvmModel::save_to_file(string path) {
    std::ofstream fs(path.c_str(), std::ios_base::out | std::ios_base::trunc);
    CHECK(fs.is_open()) << "create file " << path << "failed";
    fs << save_to_string();
}

// LibSVM-compatible text, byte for byte the reference's layout (svmmodel.cpp:193-264): header values
// with the stream's default precision, coefficients with 16 and feature values with 8 digits.
string SvmModel::save_to_string() {
    std::ostringstream s;
    s << "svm_type " << SvmParam::svm_type_name[param.svm_type] << std::endl;
    s << "kernel_type " << SvmParam::kernel_type_name[param.kernel_type] << std::endl;
    const bool poly = param.kernel_type == SvmParam::POLY, sig = param.kernel_type == SvmParam::SIGMOID;
    if (poly) s << "degree " << param.degree << std::endl;
    if (poly || sig || param.kernel_type == SvmParam::RBF) s << "gamma " << param.gamma << std::endl;
    if (poly || sig) s << "coef0 " << param.coef0 << std::endl;
    s << "nr_class " << n_classes << std::endl;
    s << "total_sv " << sv.size() << std::endl;
    s << "rho ";
    for (size_t i = 0; i < n_binary_models; ++i) s << rho.host_data()[i] << " ";
    s << std::endl;
    if (param.svm_type == SvmParam::NU_SVC || param.svm_type == SvmParam::C_SVC) {
        s << "label ";
        for (int i = 0; i < n_classes; ++i) s << label[i] << " ";
        s << std::endl << "nr_sv ";
        for (int i = 0; i < n_classes; ++i) s << n_sv.host_data()[i] << " ";
        s << std::endl;
    }
    if (param.probability == 1) {
        s << "probA ";
        for (size_t i = 0; i < n_binary_models; ++i) s << probA[i] << " ";
        s << std::endl << "probB ";
        for (size_t i = 0; i < n_binary_models; ++i) s << probB[i] << " ";
        s << std::endl;
    }
    if (param.kernel_type == SvmParam::LINEAR) {
        s << "coef " << std::endl;
        for (size_t i = 0; i < linear_coef.size(); ++i) s << std::setprecision(16) << linear_coef.host_data()[i] << " ";
        s << std::endl;
    }
    s << "SV " << std::endl;
    const float_type *cf = coef.host_data();
    for (size_t i = 0; i < sv.size(); ++i) {
        for (int j = 0; j < n_classes - 1; ++j) s << std::setprecision(16) << cf[j * sv.size() + i] << " ";
        for (auto &nd : sv[i]) s << nd.index << ":" << std::setprecision(8) << nd.value << " ";
        s << std::endl;
    }
    return s.str();
}

void SvmModel::load_from_file(string path) {
    std::ifstream ifs(path.c_str());
    if (!ifs.is_open()) {
        LOG(INFO) << "file " << path << " not found";
        exit(1);
    }
    std::stringstream ss;
    ss << ifs.rdbuf();
    load_from_string(ss.str());
}

void SvmModel::load_from_string(string data) {
    std::stringstream in(data);
    string key;
    auto lookup = [](const string &v, const char *const *names) {
        for (int i = 0; i < 5; ++i) if (v == names[i]) return i;
        return 0;
    };
    while (in >> key) {
        if (key == "svm_type") { string v; in >> v; param.svm_type = (SvmParam::SVM_TYPE) lookup(v, SvmParam::svm_type_name); }
        else if (key == "kernel_type") { string v; in >> v; param.kernel_type = (SvmParam::KERNEL_TYPE) lookup(v, SvmParam::kernel_type_name); }
        else if (key == "degree") in >> param.degree;
        else if (key == "gamma") in >> param.gamma;
        else if (key == "coef0") in >> param.coef0;
        else if (key == "nr_class") {
            in >> n_classes;
            n_binary_models = (size_t) n_classes * (n_classes - 1) / 2;
            rho.resize(n_binary_models);
            n_sv.resize(n_classes);
        } else if (key == "total_sv") in >> n_total_sv;
        else if (key == "rho") { for (size_t i = 0; i < n_binary_models; ++i) in >> rho.host_data()[i]; }
        else if (key == "label") { label.assign(n_classes, 0); for (int i = 0; i < n_classes; ++i) in >> label[i]; }
        else if (key == "nr_sv") { for (int i = 0; i < n_classes; ++i) in >> n_sv.host_data()[i]; }
        else if (key == "probA") { param.probability = 1; probA.assign(n_binary_models, 0); for (auto &v : probA) in >> v; }
        else if (key == "probB") { probB.assign(n_binary_models, 0); for (auto &v : probB) in >> v; }
        else if (key == "coef") {
            string line;
            std::getline(in, line);
            std::getline(in, line);
            std::stringstream ls(line);
            vector<float_type> w;
            float_type v;
            while (ls >> v) w.push_back(v);
            linear_coef.resize(w.size());
            if (!w.empty()) linear_coef.copy_from(w.data(), w.size());
        } else if (key == "SV") {
            sv.clear();
            invalidate_sv_matrix();
            coef.resize((size_t) (n_classes - 1) * n_total_sv);
            float_type *cf = coef.host_data();
            string line;
            std::getline(in, line);
            for (int i = 0; i < n_total_sv; ++i) {
                std::getline(in, line);
                const char *p = line.c_str();
                char *q = nullptr;
                for (int j = 0; j < n_classes - 1; ++j) { cf[(size_t) j * n_total_sv + i] = strtod(p, &q); p = q; }
                sv.emplace_back();
                for (;;) {
                    while (*p && isspace((unsigned char) *p)) ++p;
                    if (!*p) break;
                    const long idx = strtol(p, &q, 10);
                    CHECK(q != p && *q == ':') << "error when loading model file";
                    p = q + 1;
                    const float v = strtof(p, &q);
                    p = q;
                    sv.back().emplace_back((int) idx, v);
                    if (idx > sv_max_index) sv_max_index = (int) idx;
                }
            }
        }
    }
    if (param.svm_type != SvmParam::C_SVC && param.svm_type != SvmParam::NU_SVC) {
        n_sv.host_data()[0] = n_total_sv;
        n_sv.host_data()[1] = 0;
    }
}

int SvmModel::total_sv() const { return n_total_sv; }
int SvmModel::get_n_classes() const { return n_classes; }
const DataSet::node2d &SvmModel::svs() const { return sv; }
const SyncArray<int> &SvmModel::get_n_sv() const { return n_sv; }
const SyncArray<float_type> &SvmModel::get_coef() const { return coef; }
const SyncArray<float_type> &SvmModel::get_linear_coef() const { return linear_coef; }
const SyncArray<float_type> &SvmModel::get_rho() const { return rho; }
void SvmModel::set_max_iter(int iter) { max_iter = iter; }
const SyncArray<float_type> &SvmModel::get_dec_value() const { return dec_values; }
void SvmModel::set_max_memory_size(size_t size) { if (size > 0) param.max_mem_size = size << 20; }
void SvmModel::set_max_memory_size_Byte(size_t size) { if (size > 0) param.max_mem_size = size; }
int SvmModel::get_n_binary_models() const { return (int) n_binary_models; }
const vector<float> &SvmModel::get_prob_predict() const { return prob_predict; }
int SvmModel::get_sv_max_index() const { return sv_max_index; }
const vector<int> &SvmModel::get_sv_ind() const { return sv_indices; }
const vector<int> &SvmModel::get_label() const { return label; }
const bool SvmModel::is_prob() const { return param.probability; }

void SvmModel::get_param(char *kernel_type, int *degree, float *gamma, float *coef0, int *probability) {
    strcpy(kernel_type, SvmParam::kernel_type_name[param.kernel_type]);
    *degree = param.degree;
    *gamma = (float) param.gamma;
    *coef0 = (float) param.coef0;
    *probability = param.probability;
}

void SvmModel::compute_linear_coef_single_model(size_t n_feature, const bool zero_based) {
    linear_coef.resize(zero_based ? n_feature + 1 : n_feature);
    float_type *w = linear_coef.host_data();
    const float_type *cf = coef.host_data();
    for (int i = 0; i < n_total_sv; ++i)
        for (auto &nd : sv[i]) w[zero_based ? nd.index : nd.index - 1] += cf[i] * nd.value;
}

// ------------------------------------------------------------------------------------------------
// SVC / NuSVC
// ------------------------------------------------------------------------------------------------
void SVC::model_setup(const DataSet &dataset, SvmParam &param) {
    n_classes = (int) dataset.n_classes();
    LOG(INFO) << "#classes = " << n_classes;
    this->label = dataset.label();
    SvmModel::model_setup(dataset, param);
    this->param.svm_type = SvmParam::C_SVC;
    c_weight.assign(n_classes, 1);
    for (int i = 0; i < param.nr_weight; ++i) {
        bool found = false;
        for (int j = 0; j < n_classes && !found; ++j)
            if (param.weight_label[i] == dataset.label()[j]) { c_weight[j] *= param.weight[i]; found = true; }
        if (!found) LOG(WARNING) << "weighted label " << param.weight_label[i] << " not found";
    }
}

// Same storage rule as KernelMatrix (dense unless very sparse or too large), applied to the whole grouped data
// set; rows are laid out in grouped order so that every class is one contiguous block.
void SVC::build_device_rows(const DataSet &ds) {
    free_device_rows();
    const size_t n = ds.n_instances();
    if (n == 0) return;
    size_t nnz = 0;
    int mx = 0;
    {
        const DataSet::node2d &all = ds.instances();
#pragma omp parallel for schedule(static) reduction(+ : nnz) reduction(max : mx)
        for (long r = 0; r < (long) all.size(); ++r) {
            nnz += all[r].size();
            for (auto &nd : all[r]) if (nd.index > mx) mx = nd.index;
        }
    }
    const size_t d = (size_t) mx + 1, ld = (d + 3) & ~(size_t) 3;
    const double density = (double) nnz / ((double) n * d);
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    const double bytes = 4.0 * n * ld * 4.0 + 1024.0 * n * 4.0;      // this copy + a pair's matrix and planes + rows
    if (!((density >= 0.02 || d <= 256) && bytes < 0.6 * (double) free_b)) return;
    vector<float> X(n * ld, 0.0f);
    const vector<int> perm = ds.original_index();
    const DataSet::node2d &ins = ds.instances();
#pragma omp parallel for schedule(static)
    for (long k = 0; k < (long) n; ++k)
        for (auto &nd : ins[perm[k]]) X[(size_t) k * ld + nd.index] = nd.value;
    dev_rows_.X = static_cast<float *>(thundersvm::device_alloc(n * ld * sizeof(float)));
    thundersvm::copy_to_device(dev_rows_.X, X.data(), n * ld * sizeof(float));
    dev_rows_.n = n; dev_rows_.d = d; dev_rows_.ld = ld;
}

void SVC::free_device_rows() {
    thundersvm::device_free(dev_rows_.X);
    dev_rows_ = DeviceRows();
}

void SVC::train(const DataSet &dataset, SvmParam param) {
    DataSet ds = dataset;
    ds.group_classes();
    model_setup(ds, param);
    if (n_classes > 2) build_device_rows(ds);       // two classes: one sub-problem, nothing to share
    vector<std::unique_ptr<SyncArray<float_type>>> alpha(n_binary_models);
    vector<char> is_sv(ds.n_instances(), 0);
    vector<std::pair<int, int>> pairs;
    for (int i = 0; i < n_classes; ++i)
        for (int j = i + 1; j < n_classes; ++j) pairs.emplace_back(i, j);
    for (auto &a : alpha) a.reset(new SyncArray<float_type>());
    float_type *rho_h = rho.host_data();
    // The binary problems are independent (svc.cpp:50-61 solves them one after the other). With the data set on
    // the device, a few host threads take them from a common counter, each with a CUDA stream of its own, so
    // that the short launches and host waits of one solve fill the gaps of another; the model does not depend
    // on the order. THUNDERSVM_PAIR_STREAMS=1 keeps the loop sequential.
    int n_threads = 1;
    if (dev_rows_.X && pairs.size() > 1) {
        const char *e = getenv("THUNDERSVM_PAIR_STREAMS");
        n_threads = e ? atoi(e) : 4;
        if (n_threads < 1) n_threads = 1;
        if (n_threads > (int) pairs.size()) n_threads = (int) pairs.size();
    }
    if (n_threads <= 1) {
        for (size_t k = 0; k < pairs.size(); ++k) train_binary(ds, pairs[k].first, pairs[k].second, *alpha[k], rho_h[k]);
    } else {
        int dev = 0;
        cudaGetDevice(&dev);
        std::atomic<size_t> next{0};
        std::mutex err_mu;
        std::exception_ptr err;
        vector<std::thread> pool;
        for (int t = 0; t < n_threads; ++t)
            pool.emplace_back([&, dev]() {
                cudaSetDevice(dev);
                cudaStream_t s = nullptr;
                if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) s = nullptr;
                thundersvm::set_work_stream(s);
                try {
                    for (size_t k = next++; k < pairs.size(); k = next++)
                        train_binary(ds, pairs[k].first, pairs[k].second, *alpha[k], rho_h[k]);
                } catch (...) {
                    std::lock_guard<std::mutex> lk(err_mu);
                    if (!err) err = std::current_exception();
                    next = pairs.size();            // the other workers stop after their current pair
                }
                if (s) { cudaStreamSynchronize(s); cudaStreamDestroy(s); }
                thundersvm::set_work_stream(nullptr);
            });
        for (auto &th : pool) th.join();
        if (err) std::rethrow_exception(err);
    }
    for (size_t k = 0; k < pairs.size(); ++k) {
        const vector<int> ids = ds.original_index(pairs[k].first, pairs[k].second);
        CHECK_EQ(ids.size(), alpha[k]->size());
        const float_type *a = alpha[k]->host_data();
        for (size_t l = 0; l < ids.size(); ++l) if (a[l] != 0) is_sv[ids[l]] = 1;
    }
    free_device_rows();
    // support vectors in class order; n_sv per class
    int *cnt = n_sv.host_data();
    for (int c = 0; c < n_classes; ++c) {
        cnt[c] = 0;
        for (int id : ds.original_index(c))
            if (is_sv[id]) { cnt[c]++; sv.push_back(ds.instances()[id]); sv_indices.push_back(id); }
    }
    n_total_sv = (int) sv.size();
    LOG(INFO) << "#total unique sv = " << n_total_sv;
    coef.resize((size_t) (n_classes - 1) * n_total_sv);
    vector<int> sv_start(n_classes, 0);
    for (int c = 1; c < n_classes; ++c) sv_start[c] = sv_start[c - 1] + cnt[c - 1];
    // coefficient layout (svmmodel.h:155-164): pair (i, j) writes class i's alphas into row j-1 and
    // class j's into row i, at the classes' support-vector positions
    float_type *cf = coef.host_data();
    int k = 0;
    for (int i = 0; i < n_classes; ++i)
        for (int j = i + 1; j < n_classes; ++j, ++k) {
            const float_type *a = alpha[k]->host_data();
            const vector<int> ids = ds.original_index(i, j);
            const int ci = ds.count()[i], cj = ds.count()[j];
            int pos = sv_start[i];
            for (int l = 0; l < ci; ++l) if (is_sv[ids[l]]) cf[(size_t) (j - 1) * n_total_sv + pos++] = a[l];
            pos = sv_start[j];
            for (int l = ci; l < ci + cj; ++l) if (is_sv[ids[l]]) cf[(size_t) i * n_total_sv + pos++] = a[l];
        }
    if (param.kernel_type == SvmParam::LINEAR) {
        const bool zb = ds.is_zero_based();
        const size_t width = ds.n_features();
        linear_coef.resize(n_binary_models * (zb ? width + 1 : width));
        float_type *w = linear_coef.host_data();
        k = 0;
        for (int i = 0; i < n_classes; ++i)
            for (int j = i + 1; j < n_classes; ++j, ++k) {
                const float_type *a = alpha[k]->host_data();
                const DataSet::node2d ins = ds.instances(i, j);
                for (size_t r = 0; r < ins.size(); ++r)
                    if (a[r] != 0)
                        for (auto &nd : ins[r]) w[k * width + (zb ? nd.index : nd.index - 1)] += a[r] * nd.value;
            }
    }
    if (param.probability == 1) {
        LOG(INFO) << "performing probability train";
        probA.assign(n_binary_models, 0);
        probB.assign(n_binary_models, 0);
        probability_train(ds);
    }
}

void SVC::train_binary(const DataSet &dataset, int i, int j, SyncArray<float_type> &alpha, float_type &rho) {
    const int ci = dataset.count()[i], cj = dataset.count()[j];
    const size_t n_pair = (size_t) ci + cj;
    SyncArray<int> y(n_pair);
    SyncArray<float_type> f_val(n_pair);
    alpha.resize(n_pair);
    alpha.mem_set(0);
    for (int l = 0; l < ci + cj; ++l) {
        y.host_data()[l] = l < ci ? +1 : -1;
        f_val.host_data()[l] = l < ci ? -1 : +1;
    }
    std::unique_ptr<KernelMatrix> k_mat_ptr;
    if (dev_rows_.X)
        k_mat_ptr.reset(new KernelMatrix(dev_rows_.X, dev_rows_.d, dev_rows_.ld, dataset.start()[i], ci, dataset.start()[j],
                                         cj, param));
    else
        k_mat_ptr.reset(new KernelMatrix(dataset.instances(i, j), param));
    KernelMatrix &k_mat = *k_mat_ptr;
    const int ws_size = get_working_set_size((int) n_pair, (int) k_mat.n_features());
    CSMOSolver solver;
    solver.solve(k_mat, y, alpha, rho, f_val, param.epsilon, param.C * c_weight[i], param.C * c_weight[j], ws_size,
                 max_iter);
    LOG(INFO) << "rho = " << rho;
    int n_sv_pair = 0;
    float_type *a = alpha.host_data();
    const int *yy = y.host_data();
    for (size_t l = 0; l < alpha.size(); ++l) { a[l] *= yy[l]; n_sv_pair += a[l] != 0; }
    LOG(INFO) << "#sv = " << n_sv_pair;
}

void NuSVC::model_setup(const DataSet &dataset, SvmParam &param) {
    SVC::model_setup(dataset, param);
    this->param.svm_type = SvmParam::NU_SVC;
}

void NuSVC::train_binary(const DataSet &dataset, int i, int j, SyncArray<float_type> &alpha, float_type &rho) {
    const int n_pos = dataset.count()[i], n_neg = dataset.count()[j];
    const size_t n_pair = (size_t) n_pos + n_neg;
    SyncArray<int> y(n_pair);
    SyncArray<float_type> f_val(n_pair);
    alpha.resize(n_pair);
    f_val.mem_set(0);
    // nusvc.cpp:16-28: nu * n / 2 of alpha mass per class, filled from the front
    float_type budget_p = param.nu * n_pair / 2, budget_n = budget_p;
    float_type *a = alpha.host_data();
    int *yy = y.host_data();
    for (int l = 0; l < n_pos; ++l) { yy[l] = +1; a[l] = std::min(1., budget_p); budget_p -= a[l]; }
    for (int l = n_pos; l < n_pos + n_neg; ++l) { yy[l] = -1; a[l] = std::min(1., budget_n); budget_n -= a[l]; }
    std::unique_ptr<KernelMatrix> k_mat_ptr;
    if (dev_rows_.X)
        k_mat_ptr.reset(new KernelMatrix(dev_rows_.X, dev_rows_.d, dev_rows_.ld, dataset.start()[i], n_pos,
                                         dataset.start()[j], n_neg, param));
    else
        k_mat_ptr.reset(new KernelMatrix(dataset.instances(i, j), param));
    KernelMatrix &k_mat = *k_mat_ptr;
    const int ws_size = get_working_set_size((int) n_pair, (int) k_mat.n_features());
    NuSMOSolver solver(false);
    solver.solve(k_mat, y, alpha, rho, f_val, param.epsilon, 1, 1, ws_size, max_iter);
    LOG(INFO) << "rho = " << rho;
    int n_sv_pair = 0;
    a = alpha.host_data();
    yy = y.host_data();
    for (size_t l = 0; l < alpha.size(); ++l) { a[l] *= yy[l]; n_sv_pair += a[l] != 0; }
    LOG(INFO) << "#sv = " << n_sv_pair;
}

vector<float_type> SVC::predict(const DataSet::node2d &instances, int batch_size) {
    if (n_binary_models > 10000) return predict_instant(instances, batch_size);
    dec_values.resize(instances.size() * n_binary_models);
    predict_dec_values(instances, dec_values, batch_size);
    return predict_label(dec_values, (int) instances.size());
}

vector<float_type> SVC::predict_instant(const DataSet::node2d &instances, int batch_size) {
    SyncArray<float_type> idx(instances.size());
    predict_dec_values_instant(instances, idx, batch_size);
    vector<float_type> out(instances.size());
    for (size_t i = 0; i < out.size(); ++i) out[i] = (double) label[(int) idx.host_data()[i]];
    return out;
}

// Platt's sigmoid in the numerically careful form: 1 / (1 + exp(A f + B))
static float_type sigmoid_predict(float_type dec, float_type A, float_type B) {
    const double t = dec * A + B;
    return t >= 0 ? exp(-t) / (1.0 + exp(-t)) : 1.0 / (1 + exp(t));
}

// Pairwise coupling (Wu, Lin and Weng, 2004, second method): minimise sum_{i != j} (r_ji p_i - r_ij p_j)^2
// over the simplex by the fixed-point iteration of their Algorithm 2.
void SVC::multiclass_probability(const vector<vector<float_type>> &r, vector<float_type> &p) const {
    const int k = n_classes;
    const int max_it = std::max(100, k);
    const double eps = 0.005 / k;
    vector<vector<double>> Q(k, vector<double>(k, 0.0));
    vector<double> Qp(k);
    for (int t = 0; t < k; ++t) {
        p[t] = 1.0 / k;
        for (int j = 0; j < k; ++j) {
            if (j == t) continue;
            Q[t][t] += r[j][t] * r[j][t];
            Q[t][j] = -r[j][t] * r[t][j];
        }
    }
    int it = 0;
    for (; it < max_it; ++it) {
        double pQp = 0;
        for (int t = 0; t < k; ++t) {
            Qp[t] = 0;
            for (int j = 0; j < k; ++j) Qp[t] += Q[t][j] * p[j];
            pQp += p[t] * Qp[t];
        }
        double worst = 0;
        for (int t = 0; t < k; ++t) worst = std::max(worst, fabs(Qp[t] - pQp));
        if (worst < eps) break;
        for (int t = 0; t < k; ++t) {
            const double diff = (-Qp[t] + pQp) / Q[t][t];
            p[t] += diff;
            pQp = (pQp + diff * (diff * Q[t][t] + 2 * Qp[t])) / (1 + diff) / (1 + diff);
            for (int j = 0; j < k; ++j) {
                Qp[j] = (Qp[j] + diff * Q[t][j]) / (1 + diff);
                p[j] /= (1 + diff);
            }
        }
    }
    if (it >= max_it) printf("Exceeds max_iter in multiclass_prob\n");
}

vector<float_type> SVC::predict_label(const SyncArray<float_type> &dec_values, int n_instances) {
    vector<float_type> out;
    out.reserve(n_instances);
    const float_type *d = dec_values.host_data();
    if (param.probability == 0) {
        vector<int> votes(n_classes);
        for (int r = 0; r < n_instances; ++r) {
            std::fill(votes.begin(), votes.end(), 0);
            int k = 0;
            for (int i = 0; i < n_classes; ++i)
                for (int j = i + 1; j < n_classes; ++j, ++k) votes[d[(size_t) r * n_binary_models + k] > 0 ? i : j]++;
            int best = 0;
            for (int c = 1; c < n_classes; ++c) if (votes[c] > votes[best]) best = c;
            out.push_back((float) label[best]);
        }
        return out;
    }
    LOG(INFO) << "predict with probability";
    prob_predict.clear();
    const float_type min_prob = 1e-7;
    for (int r = 0; r < n_instances; ++r) {
        vector<vector<float_type>> pair(n_classes, vector<float_type>(n_classes));
        int k = 0;
        for (int i = 0; i < n_classes; ++i)
            for (int j = i + 1; j < n_classes; ++j, ++k) {
                const float_type v = sigmoid_predict(d[(size_t) r * n_binary_models + k], probA[k], probB[k]);
                pair[i][j] = std::min(std::max(v, min_prob), 1 - min_prob);
                pair[j][i] = 1 - pair[i][j];
            }
        vector<float_type> p(n_classes);
        multiclass_probability(pair, p);
        prob_predict.insert(prob_predict.end(), p.begin(), p.end());
        int best = 0;
        for (int c = 1; c < n_classes; ++c) if (p[c] > p[best]) best = c;
        out.push_back((float) label[best]);
    }
    return out;
}

// Fits P(y = 1 | f) = 1 / (1 + exp(A f + B)) by the Newton method with backtracking of Lin, Lin and Weng
// (2007), the algorithm LibSVM and the reference (svc.cpp:318-425) use.
static void sigmoid_train(const vector<float_type> &dec, const vector<int> &labels, float_type &A, float_type &B) {
    const int l = (int) dec.size();
    double n_pos = 0, n_neg = 0;
    for (int i = 0; i < l; ++i) (labels[i] > 0 ? n_pos : n_neg) += 1;
    const int max_it = 100;
    const double min_step = 1e-10, sigma = 1e-12, tol = 1e-5;
    const double hi = (n_pos + 1.0) / (n_pos + 2.0), lo = 1 / (n_neg + 2.0);
    vector<double> t(l);
    A = 0.0;
    B = log((n_neg + 1.0) / (n_pos + 1.0));
    auto objective = [&](double a, double b) {
        double f = 0;
        for (int i = 0; i < l; ++i) {
            const double z = dec[i] * a + b;
            f += z >= 0 ? t[i] * z + log(1 + exp(-z)) : (t[i] - 1) * z + log(1 + exp(z));
        }
        return f;
    };
    for (int i = 0; i < l; ++i) t[i] = labels[i] > 0 ? hi : lo;
    double fval = objective(A, B);
    int it = 0;
    for (; it < max_it; ++it) {
        double h11 = sigma, h22 = sigma, h21 = 0, g1 = 0, g2 = 0;
        for (int i = 0; i < l; ++i) {
            const double z = dec[i] * A + B;
            double p, q;
            if (z >= 0) { p = exp(-z) / (1.0 + exp(-z)); q = 1.0 / (1.0 + exp(-z)); }
            else { p = 1.0 / (1.0 + exp(z)); q = exp(z) / (1.0 + exp(z)); }
            const double d2 = p * q, d1 = t[i] - p;
            h11 += dec[i] * dec[i] * d2; h22 += d2; h21 += dec[i] * d2;
            g1 += dec[i] * d1; g2 += d1;
        }
        if (fabs(g1) < tol && fabs(g2) < tol) break;
        const double det = h11 * h22 - h21 * h21;
        const double dA = -(h22 * g1 - h21 * g2) / det, dB = -(-h21 * g1 + h11 * g2) / det;
        const double gd = g1 * dA + g2 * dB;
        double step = 1;
        while (step >= min_step) {
            const double nA = A + step * dA, nB = B + step * dB, nf = objective(nA, nB);
            if (nf < fval + 0.0001 * step * gd) { A = nA; B = nB; fval = nf; break; }
            step /= 2.0;
        }
        if (step < min_step) { printf("Line search fails in two-class probability estimates\n"); break; }
    }
    if (it >= max_it) printf("Reaching maximal iterations in two-class probability estimates\n");
}

void SVC::probability_train(const DataSet &dataset) {
    SvmParam plain = param;
    plain.probability = 0;
    vector<float_type> dec_all(dataset.n_instances() * n_binary_models);
    const int n_fold = 5;
    for (int k = 0; k < n_fold; ++k) {
        DataSet::node2d x_train, x_test;
        vector<float_type> y_train, y_test;
        vector<int> test_idx;
        fold_split(dataset, n_fold, k, x_train, y_train, x_test, y_test, test_idx);
        std::unique_ptr<SvmModel> fold_model(new SVC());
        DataSet train_set(x_train, (int) dataset.n_features(), y_train);
        fold_model->train(train_set, plain);
        SyncArray<float_type> dec(x_test.size() * n_binary_models);
        fold_model->predict_dec_values(x_test, dec, 1000);
        const float_type *d = dec.host_data();
        for (size_t i = 0; i < x_test.size(); ++i)
            memcpy(&dec_all[test_idx[i] * n_binary_models], &d[i * n_binary_models], sizeof(float_type) * n_binary_models);
    }
    int k = 0;
    for (int i = 0; i < n_classes; ++i)
        for (int j = i + 1; j < n_classes; ++j, ++k) {
            vector<int> y;
            vector<float_type> dec;
            for (int id : dataset.original_index(i)) { y.push_back(+1); dec.push_back(dec_all[id * n_binary_models + k]); }
            for (int id : dataset.original_index(j)) { y.push_back(-1); dec.push_back(dec_all[id * n_binary_models + k]); }
            sigmoid_train(dec, y, probA[k], probB[k]);
        }
}

// ------------------------------------------------------------------------------------------------
// SVR / NuSVR / OneClassSVC
// ------------------------------------------------------------------------------------------------
void SVR::model_setup(const DataSet &dataset, SvmParam &param) {
    SvmModel::model_setup(dataset, param);
    this->param.svm_type = SvmParam::EPSILON_SVR;
}

void SVR::save_svr_coef(const SyncArray<float_type> &alpha_2, const DataSet::node2d &instances) {
    LOG(INFO) << "rho = " << rho.host_data()[0];
    const int n = (int) alpha_2.size() / 2;
    const float_type *a = alpha_2.host_data();
    vector<float_type> cf;
    for (int i = 0; i < n; ++i) {
        const float_type v = a[i] - a[i + n];
        if (v != 0) { sv.push_back(instances[i]); sv_indices.push_back(i); cf.push_back(v); }
    }
    LOG(INFO) << "#sv = " << sv.size();
    n_sv.host_data()[0] = (int) sv.size();
    n_sv.host_data()[1] = 0;
    n_total_sv = (int) sv.size();
    coef.resize(std::max<size_t>(cf.size(), 0));
    if (!cf.empty()) coef.copy_from(cf.data(), cf.size());
}

void SVR::train(const DataSet &dataset, SvmParam param) {
    model_setup(dataset, param);
    const int n = (int) dataset.n_instances();
    DataSet::node2d twice(dataset.instances());                 // the dual runs over 2n duplicated instances
    twice.insert(twice.end(), dataset.instances().begin(), dataset.instances().end());
    KernelMatrix k_mat(twice, param);
    SyncArray<float_type> f_val(2 * n), alpha_2(2 * n);
    SyncArray<int> y(2 * n);
    alpha_2.mem_set(0);
    for (int i = 0; i < n; ++i) {
        f_val.host_data()[i] = param.p - dataset.y()[i];
        y.host_data()[i] = +1;
        f_val.host_data()[i + n] = -param.p - dataset.y()[i];
        y.host_data()[i + n] = -1;
    }
    const int ws_size = get_working_set_size(2 * n, (int) k_mat.n_features());
    CSMOSolver solver;
    solver.solve(k_mat, y, alpha_2, rho.host_data()[0], f_val, param.epsilon, param.C, param.C, ws_size, max_iter);
    save_svr_coef(alpha_2, dataset.instances());
    if (param.kernel_type == SvmParam::LINEAR) compute_linear_coef_single_model(dataset.n_features(), dataset.is_zero_based());
}

void NuSVR::model_setup(const DataSet &dataset, SvmParam &param) {
    SVR::model_setup(dataset, param);
    this->param.svm_type = SvmParam::NU_SVR;
}

void NuSVR::train(const DataSet &dataset, SvmParam param) {
    model_setup(dataset, param);
    const int n = (int) dataset.n_instances();
    DataSet::node2d twice(dataset.instances());
    twice.insert(twice.end(), dataset.instances().begin(), dataset.instances().end());
    KernelMatrix k_mat(twice, param);
    SyncArray<float_type> f_val(2 * n), alpha_2(2 * n);
    SyncArray<int> y(2 * n);
    float_type mass = param.C * param.nu * n / 2;               // nusvr.cpp:24-32
    for (int i = 0; i < n; ++i) {
        const float_type a = std::min(mass, param.C);
        alpha_2.host_data()[i] = alpha_2.host_data()[i + n] = a;
        mass -= a;
        f_val.host_data()[i] = f_val.host_data()[i + n] = -dataset.y()[i];
        y.host_data()[i] = +1;
        y.host_data()[i + n] = -1;
    }
    const int ws_size = get_working_set_size(2 * n, (int) k_mat.n_features());
    NuSMOSolver solver(true);
    solver.solve(k_mat, y, alpha_2, rho.host_data()[0], f_val, param.epsilon, param.C, param.C, ws_size, max_iter);
    save_svr_coef(alpha_2, dataset.instances());
    if (param.kernel_type == SvmParam::LINEAR) compute_linear_coef_single_model(dataset.n_features(), dataset.is_zero_based());
}

void OneClassSVC::model_setup(const DataSet &dataset, SvmParam &param) {
    SvmModel::model_setup(dataset, param);
    this->param.svm_type = SvmParam::ONE_CLASS;
}

void OneClassSVC::train(const DataSet &dataset, SvmParam param) {
    model_setup(dataset, param);
    const int n = (int) dataset.n_instances();
    SyncArray<float_type> alpha(n), f_val(n);
    SyncArray<int> y(n);
    KernelMatrix k_mat(dataset.instances(), param);
    alpha.mem_set(0);
    f_val.mem_set(0);
    const int full = static_cast<int>(param.nu * n);            // oneclass_svc.cpp:18-24
    for (int i = 0; i < full; ++i) alpha.host_data()[i] = 1;
    if (full < n) alpha.host_data()[full] = param.nu * n - full;
    for (int i = 0; i < n; ++i) y.host_data()[i] = 1;
    const int ws_size = get_working_set_size(n, (int) k_mat.n_features());
    CSMOSolver solver;
    solver.solve(k_mat, y, alpha, rho.host_data()[0], f_val, param.epsilon, 1, 1, ws_size, max_iter);
    LOG(INFO) << "rho = " << rho.host_data()[0];
    vector<float_type> cf;
    const float_type *a = alpha.host_data();
    for (int i = 0; i < n; ++i)
        if (a[i] != 0) { sv.push_back(dataset.instances()[i]); sv_indices.push_back(i); cf.push_back(a[i]); }
    LOG(INFO) << "#sv = " << sv.size();
    n_sv.host_data()[0] = (int) sv.size();
    n_sv.host_data()[1] = 0;
    n_total_sv = (int) sv.size();
    coef.resize(cf.size());
    if (!cf.empty()) coef.copy_from(cf.data(), cf.size());
    if (param.kernel_type == SvmParam::LINEAR) compute_linear_coef_single_model(dataset.n_features(), dataset.is_zero_based());
}

vector<float_type> OneClassSVC::predict(const DataSet::node2d &instances, int batch_size) {
    vector<float_type> dec = SvmModel::predict(instances, batch_size);
    for (auto &v : dec) v = v > 0 ? 1 : -1;
    return dec;
}
