// DataSet loaders and class grouping. Behaviour follows src/thundersvm/dataset.cpp:20-291: LibSVM
// text keeps its 1-based feature ids (a 0 id flags the set as zero based), CSR input is shifted to
// 1-based, dense input numbers its columns 1..d and keeps explicit zeros; group_classes orders the
// classes by first appearance and records the permutation.
#include <thundersvm/dataset.h>
#include <cstdio>
#include <fstream>

DataSet::DataSet() : rows_(std::make_shared<node2d>()), total_count_(0), n_features_(0) {}

DataSet::DataSet(const DataSet::node2d &instances, int n_features, const vector<float_type> &y)
    : y_(y), rows_(std::make_shared<node2d>(instances)), total_count_(instances.size()), n_features_(n_features) {}

namespace {
// parses one "label idx:val idx:val ..." line in place; returns false for blank lines
bool parse_line(const char *p, const char *end, float_type &label, vector<DataSet::node> &row, bool &saw_zero,
                size_t &max_index) {
    while (p < end && isspace((unsigned char) *p)) ++p;
    if (p >= end) return false;
    char *q = nullptr;
    label = strtod(p, &q);
    CHECK(q != p) << "read error: a line must start with a label";
    p = q;
    for (;;) {
        while (p < end && isspace((unsigned char) *p)) ++p;
        if (p >= end) break;
        long idx = strtol(p, &q, 10);
        CHECK(q != p && *q == ':') << "read error, using [index]:[value] format";
        p = q + 1;
        float v = strtof(p, &q);
        CHECK(q != p) << "read error, using [index]:[value] format";
        p = q;
        row.emplace_back((int) idx, v);
        if (idx == 0) saw_zero = true;
        if ((size_t) idx > max_index) max_index = idx;
    }
    return true;
}
}  // namespace

void DataSet::load_from_file(string file_name) {
    LOG(INFO) << "loading dataset from file \"" << file_name << "\"";
    rows_ = std::make_shared<node2d>();
    node2d &instances_ = *rows_;
    y_.clear(); total_count_ = 0; n_features_ = 0;
    std::ifstream ifs(file_name, std::ifstream::binary);
    if (!ifs.is_open()) {
        LOG(INFO) << "file " << file_name << " not found";
        exit(1);
    }
    string text((std::istreambuf_iterator<char>(ifs)), std::istreambuf_iterator<char>());
    // line starts, then the lines are parsed in parallel into their final slots
    vector<size_t> starts(1, 0);
    for (size_t i = 0; i < text.size(); ++i)
        if (text[i] == '\n') starts.push_back(i + 1);
    if (starts.back() != text.size()) starts.push_back(text.size() + 1);
    const long n_lines = (long) starts.size() - 1;
    vector<vector<node>> rows(n_lines);
    vector<float_type> labels(n_lines);
    vector<char> used(n_lines, 0);
    bool saw_zero = false;
    size_t max_index = 0;
#pragma omp parallel for schedule(dynamic, 256) reduction(|| : saw_zero) reduction(max : max_index)
    for (long l = 0; l < n_lines; ++l) {
        const char *b = text.data() + starts[l];
        const char *e = text.data() + std::min(starts[l + 1] - 1, text.size());
        used[l] = parse_line(b, e, labels[l], rows[l], saw_zero, max_index);
    }
    for (long l = 0; l < n_lines; ++l)
        if (used[l]) { y_.push_back(labels[l]); instances_.emplace_back(std::move(rows[l])); }
    total_count_ = instances_.size();
    n_features_ = max_index;
    zero_based = saw_zero;
    LOG(INFO) << "#instances = " << n_instances() << ", #features = " << n_features();
}

void DataSet::load_from_python(float *y, char **x, int len) {
    rows_ = std::make_shared<node2d>();
    node2d &instances_ = *rows_;
    y_.clear(); total_count_ = 0; n_features_ = 0;
    bool saw_zero = false;
    size_t max_index = 0;
    for (int i = 0; i < len; ++i) {
        // x[i] holds only the "idx:val ..." part of the line
        const string line = string("0 ") + x[i];
        float_type dummy;
        instances_.emplace_back();
        parse_line(line.data(), line.data() + line.size(), dummy, instances_.back(), saw_zero, max_index);
        y_.push_back(y[i]);
        total_count_++;
    }
    n_features_ = max_index;
}

void DataSet::load_from_sparse(int row_size, float *val, int *row_ptr, int *col_ptr, float *label) {
    rows_ = std::make_shared<node2d>();
    node2d &instances_ = *rows_;
    y_.clear(); total_count_ = 0; n_features_ = 0;
    instances_.resize(row_size);
    for (int r = 0; r < row_size; ++r) {
        if (label) y_.push_back(label[r]);
        auto &row = instances_[r];
        row.reserve(row_ptr[r + 1] - row_ptr[r]);
        for (int p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
            const int idx = col_ptr[p] + 1;                 // to the one-based convention
            row.emplace_back(idx, val[p]);
            if ((size_t) idx > n_features_) n_features_ = idx;
        }
    }
    total_count_ = row_size;
    LOG(INFO) << "#instances = " << n_instances() << ", #features = " << n_features();
}

void DataSet::load_from_dense(int row_size, int features, float *data, float *label) {
    rows_ = std::make_shared<node2d>();
    node2d &instances_ = *rows_;
    y_.clear(); total_count_ = 0;
    instances_.resize(row_size);
    if (label) y_.assign(label, label + row_size);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < row_size; ++r) {
        auto &row = instances_[r];
        row.reserve(features);
        const float *src = data + (size_t) r * features;
        for (int j = 0; j < features; ++j) row.emplace_back(j + 1, src[j]);     // explicit zeros are kept
    }
    total_count_ = row_size;
    n_features_ = features;
    LOG(INFO) << "#instances = " << n_instances() << ", #features = " << n_features();
}

void DataSet::group_classes(bool classification) {
    start_.clear(); count_.clear(); label_.clear(); perm_.clear();
    if (!classification) {
        perm_.resize(rows_->size());
        for (size_t i = 0; i < perm_.size(); ++i) perm_[i] = (int) i;
        start_.push_back(0);
        count_.push_back((int) rows_->size());
        return;
    }
    vector<int> cls(y_.size());
    for (size_t i = 0; i < y_.size(); ++i) {
        size_t j = 0;
        while (j < label_.size() && y_[i] != label_[j]) ++j;
        if (j == label_.size()) { label_.push_back(int(y_[i])); count_.push_back(0); }
        count_[j]++;
        cls[i] = (int) j;
    }
    start_.assign(count_.size(), 0);
    for (size_t c = 1; c < count_.size(); ++c) start_[c] = start_[c - 1] + count_[c - 1];
    vector<int> cursor(start_);
    perm_.resize(y_.size());
    for (size_t i = 0; i < y_.size(); ++i) perm_[cursor[cls[i]]++] = (int) i;
}

size_t DataSet::n_instances() const { return total_count_; }
size_t DataSet::n_features() const { return n_features_; }
size_t DataSet::n_classes() const { return start_.size(); }
const vector<int> &DataSet::count() const { return count_; }
const vector<int> &DataSet::start() const { return start_; }
const vector<int> &DataSet::label() const { return label_; }
const vector<float_type> &DataSet::y() const { return y_; }
const DataSet::node2d &DataSet::instances() const { return *rows_; }
const bool DataSet::is_zero_based() const { return zero_based; }

const DataSet::node2d DataSet::instances(int y_i) const {
    node2d out;
    out.reserve(count_[y_i]);
    for (int k = start_[y_i]; k < start_[y_i] + count_[y_i]; ++k) out.push_back((*rows_)[perm_[k]]);
    return out;
}
const DataSet::node2d DataSet::instances(int y_i, int y_j) const {
    node2d out = instances(y_i);
    node2d second = instances(y_j);
    out.insert(out.end(), second.begin(), second.end());
    return out;
}
const vector<int> DataSet::original_index() const { return perm_; }
const vector<int> DataSet::original_index(int y_i) const {
    return vector<int>(perm_.begin() + start_[y_i], perm_.begin() + start_[y_i] + count_[y_i]);
}
const vector<int> DataSet::original_index(int y_i, int y_j) const {
    vector<int> out = original_index(y_i);
    vector<int> second = original_index(y_j);
    out.insert(out.end(), second.begin(), second.end());
    return out;
}
