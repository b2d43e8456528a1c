// DataSet: LibSVM-format instances with the reference's accessors (include/thundersvm/dataset.h:14-94).
// Feature ids stay 1-based as read from LibSVM text (0-based files are detected and flagged).
#ifndef THUNDERSVM_DATASET_H
#define THUNDERSVM_DATASET_H
#include "thundersvm.h"
#include "syncarray.h"
#include <memory>

class DataSet {
public:
    struct node {
        node(int index, kernel_type value) : index(index), value(value) {}
        int index;
        kernel_type value;
    };
    typedef vector<vector<DataSet::node>> node2d;

    DataSet();
    DataSet(const DataSet::node2d &instances, int n_features, const vector<float_type> &y);

    void load_from_file(string file_name);
    void load_from_python(float *y, char **x, int len);
    void load_from_sparse(int row_size, float *val, int *row_ptr, int *col_ptr, float *label);
    void load_from_dense(int row_size, int features, float *data, float *label);
    void group_classes(bool classification = true);

    size_t n_instances() const;
    size_t n_features() const;
    size_t n_classes() const;
    const vector<int> &count() const;
    const vector<int> &start() const;
    const vector<int> &label() const;
    const vector<float_type> &y() const;
    const node2d &instances() const;
    const node2d instances(int y_i) const;
    const node2d instances(int y_i, int y_j) const;
    const vector<int> original_index() const;
    const vector<int> original_index(int y_i) const;
    const vector<int> original_index(int y_i, int y_j) const;
    const bool is_zero_based() const;

private:
    vector<float_type> y_;
    // shared between copies of a data set (a copy costs no rows): the loaders replace it, nothing edits it in place
    std::shared_ptr<node2d> rows_;
    size_t total_count_;
    size_t n_features_;
    vector<int> start_, count_, label_, perm_;
    bool zero_based = false;
};
#endif
