// Command-line style entry points kept for the Matlab / Python front ends
// (include/thundersvm/svm_interface_api.h:5-8).
#ifndef THUNDERSVM_SVM_INTERFACE_API_H
#define THUNDERSVM_SVM_INTERFACE_API_H
extern "C" {
void thundersvm_train(int argc, char **argv);
void thundersvm_train_after_parse(char **option, int len, char *file_name);
void thundersvm_predict(int argc, char **argv);
void thundersvm_predict_after_parse(char *model_file_name, char *output_file_name, char **option, int len);
void load_from_python_interface(float *y, char **x, int len);
}
#endif
