// SvmParam with the reference's fields and defaults (include/thundersvm/svmparam.h:13-68).
#ifndef THUNDERSVM_SVMPARAM_H
#define THUNDERSVM_SVMPARAM_H
#include "thundersvm.h"

struct SvmParam {
    enum SVM_TYPE { C_SVC, NU_SVC, ONE_CLASS, EPSILON_SVR, NU_SVR };
    enum KERNEL_TYPE { LINEAR, POLY, RBF, SIGMOID, PRECOMPUTED };

    SvmParam()
        : svm_type(C_SVC), kernel_type(RBF), C(1), gamma(0), p(0.1f), nu(0.5), epsilon(0.001f), degree(3), coef0(0),
          nr_weight(0), weight_label(nullptr), weight(nullptr), probability(0),
          max_mem_size(static_cast<size_t>(8192) << 20) {}

    SVM_TYPE svm_type;
    KERNEL_TYPE kernel_type;
    float_type C;          // regularisation
    float_type gamma;      // RBF / polynomial / sigmoid
    float_type p;          // epsilon of epsilon-SVR
    float_type nu;
    float_type epsilon;    // stopping tolerance
    int degree;
    float_type coef0;
    int nr_weight;         // class weights (C-SVC)
    int *weight_label;
    float_type *weight;
    int probability;
    size_t max_mem_size;   // bytes
    static const char *kernel_type_name[6];
    static const char *svm_type_name[6];
};
#endif
