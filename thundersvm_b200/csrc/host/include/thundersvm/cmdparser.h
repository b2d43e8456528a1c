// LibSVM-style option parsing for thundersvm-train / thundersvm-predict
// (include/thundersvm/cmdparser.h:17-38, src/thundersvm/cmdparser.cpp:59-355).
#ifndef THUNDERSVM_CMDPARSER_H
#define THUNDERSVM_CMDPARSER_H
#include "thundersvm.h"
#include "svmparam.h"

class CMDParser {
public:
    CMDParser() : do_cross_validation(false), gamma_set(false), nr_fold(0), gpu_id(0), n_cores(-1) {}
    void parse_command_line(int argc, char **argv);
    void parse_python(int argc, char **argv);
    bool check_parameter();

    SvmParam param_cmd;
    bool do_cross_validation;
    bool gamma_set;
    int nr_fold;
    int gpu_id;
    int n_cores;
    string svmtrain_input_file_name;
    string svmpredict_input_file;
    string svmpredict_output_file;
    string svmpredict_model_file_name;
    string model_file_name;
};
#endif
