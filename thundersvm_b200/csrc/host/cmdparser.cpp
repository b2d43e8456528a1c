// LibSVM-style option parsing (reference: src/thundersvm/cmdparser.cpp:59-355): the same letters,
// the same defaults, help text + exit(1) on malformed input.
#include <thundersvm/cmdparser.h>
#include <cstring>
#include <omp.h>

namespace {
[[noreturn]] void usage_train() {
    printf("Usage (same as LibSVM): thundersvm-train [options] training_set_file [model_file]\n"
           "options:\n"
           "-s svm_type: set type of SVM (default 0)\n"
           "	0 -- C-SVC		(multi-class classification)\n"
           "	1 -- nu-SVC		(multi-class classification)\n"
           "	2 -- one-class SVM\n"
           "	3 -- epsilon-SVR	(regression)\n"
           "	4 -- nu-SVR		(regression)\n"
           "-t kernel_type: set type of kernel function (default 2)\n"
           "	0 -- linear: u'*v\n"
           "	1 -- polynomial: (gamma*u'*v + coef0)^degree\n"
           "	2 -- radial basis function: exp(-gamma*|u-v|^2)\n"
           "	3 -- sigmoid: tanh(gamma*u'*v + coef0)\n"
           "	4 -- precomputed kernel -- not supported yet\n"
           "-d degree: set degree in kernel function (default 3)\n"
           "-g gamma: set gamma in kernel function (default 1/num_features)\n"
           "-r coef0: set coef0 in kernel function (default 0)\n"
           "-c cost: set the parameter C of C-SVC, epsilon-SVR, and nu-SVR (default 1)\n"
           "-n nu: set the parameter nu of nu-SVC, one-class SVM, and nu-SVR (default 0.5)\n"
           "-p epsilon: set the epsilon in loss function of epsilon-SVR (default 0.1)\n"
           "-m memory size: constrain the maximum memory size (MB) that thundersvm uses (default 8192)\n"
           "-e epsilon: set tolerance of termination criterion (default 0.001)\n"
           "-b probability_estimates: whether to train a SVC or SVR model for probability estimates, 0 or 1 (default 0)\n"
           "-wi weight: set the parameter C of class i to weight*C, for C-SVC (default 1)\n"
           "-v n: n-fold cross validation mode\n"
           "-u n: specify which gpu to use (default 0)\n"
           "-o n: set the number of cpu cores to use, -1 for maximum(default -1)\n"
           "-q: quiet mode\n");
    exit(1);
}
[[noreturn]] void usage_predict() {
    printf("Usage: thundersvm-predict [options] test_file model_file output_file\n"
           "options:\n"
           "-m memory size: constrain the maximum memory size (MB) that thundersvm uses (default 8192)\n"
           "-u n: specify which gpu to use (default 0)\n"
           "-o n: set the number of cpu cores to use, -1 for maximum(default -1)\n");
    exit(1);
}
double parse_gamma(const char *s) {          // "1/8" style fractions are accepted
    const char *slash = strchr(s, '/');
    return slash ? atof(string(s, slash).c_str()) / atof(slash + 1) : atof(s);
}
}  // namespace

// Shared by the CLI (first = 1, options of thundersvm-train) and the Python/Matlab string interface.
static int parse_train_options(CMDParser &P, int argc, char **argv, int first, bool &quiet) {
    int i = first;
    for (; i < argc; ++i) {
        if (argv[i][0] != '-') break;
        if (++i >= argc) usage_train();
        const char *v = argv[i];
        switch (argv[i - 1][1]) {
            case 's': P.param_cmd.svm_type = static_cast<SvmParam::SVM_TYPE>(atoi(v)); break;
            case 't': P.param_cmd.kernel_type = static_cast<SvmParam::KERNEL_TYPE>(atoi(v)); break;
            case 'd': P.param_cmd.degree = atoi(v); break;
            case 'g': P.param_cmd.gamma = parse_gamma(v); P.gamma_set = true; break;
            case 'r': P.param_cmd.coef0 = atof(v); break;
            case 'n': P.param_cmd.nu = atof(v); break;
            case 'm': P.param_cmd.max_mem_size = static_cast<size_t>(std::max(atoi(v), 0)) << 20; break;
            case 'c': P.param_cmd.C = atof(v); break;
            case 'e': P.param_cmd.epsilon = atof(v); break;
            case 'p': P.param_cmd.p = atof(v); break;
            case 'h': LOG(WARNING) << "shrinking is not supported"; break;
            case 'b': P.param_cmd.probability = atoi(v); break;
            case 'o': P.n_cores = atoi(v); break;
            case 'q': quiet = true; --i; break;
            case 'v':
                P.do_cross_validation = true;
                P.nr_fold = atoi(v);
                if (P.nr_fold < 2) { LOG(ERROR) << "n-fold cross validation: n must >= 2"; usage_train(); }
                break;
            case 'w': {
                SvmParam &p = P.param_cmd;
                ++p.nr_weight;
                p.weight_label = (int *) realloc(p.weight_label, sizeof(int) * p.nr_weight);
                p.weight = (float_type *) realloc(p.weight, sizeof(float_type) * p.nr_weight);
                p.weight_label[p.nr_weight - 1] = atoi(&argv[i - 1][2]);
                p.weight[p.nr_weight - 1] = atof(v);
                break;
            }
            case 'u': P.gpu_id = atoi(v); break;
            default:
                LOG(ERROR) << "Unknown option: " + string(argv[i - 1]);
                usage_train();
        }
    }
    if (P.n_cores > 0) omp_set_num_threads(P.n_cores);
    else if (P.n_cores != -1) LOG(ERROR) << "the number of cpu cores must be positive or -1";
    return i;
}

void CMDParser::parse_command_line(int argc, char **argv) {
    param_cmd.weight_label = nullptr;
    param_cmd.weight = nullptr;
    string bin = argv[0];
    bin = bin.substr(bin.find_last_of("/") + 1);
    bool quiet = false;
    if (bin == "thundersvm-train") {
        const int i = parse_train_options(*this, argc, argv, 1, quiet);
        if (i >= argc) usage_train();
        if (!check_parameter()) usage_train();
        svmtrain_input_file_name = argv[i];
        if (i < argc - 1) model_file_name = argv[i + 1];
        else {
            const char *slash = strrchr(argv[i], '/');
            model_file_name = string(slash ? slash + 1 : argv[i]) + ".model";
        }
    } else if (bin == "thundersvm-predict") {
        int i = 1;
        for (; i < argc; ++i) {
            if (argv[i][0] != '-') break;
            ++i;
            if (i >= argc) usage_predict();
            switch (argv[i - 1][1]) {
                case 'b': break;
                case 'u': gpu_id = atoi(argv[i]); break;
                case 'o': n_cores = atoi(argv[i]); break;
                case 'm': param_cmd.max_mem_size = static_cast<size_t>(std::max(atoi(argv[i]), 0)) << 20; break;
                default: fprintf(stderr, "Unknown option: -%c\n", argv[i - 1][1]); usage_predict();
            }
        }
        if (n_cores > 0) omp_set_num_threads(n_cores);
        else if (n_cores != -1) LOG(ERROR) << "the number of cpu cores must be positive or -1";
        if (i >= argc - 2) usage_predict();
        svmpredict_input_file = argv[i];
        svmpredict_model_file_name = argv[i + 1];
        svmpredict_output_file = argv[i + 2];
    }
    thundersvm::set_verbose(!quiet);
}

void CMDParser::parse_python(int argc, char **argv) {
    param_cmd.weight_label = nullptr;
    param_cmd.weight = nullptr;
    bool quiet = false;
    parse_train_options(*this, argc, argv, 0, quiet);
    if (!check_parameter()) usage_train();
    thundersvm::set_verbose(!quiet);
}

bool CMDParser::check_parameter() {
    const SvmParam &p = param_cmd;
    auto fail = [](const char *why) { LOG(ERROR) << why; return false; };
    if (p.svm_type < SvmParam::C_SVC || p.svm_type > SvmParam::NU_SVR) return fail("unknown svm type");
    if (p.kernel_type < SvmParam::LINEAR || p.kernel_type > SvmParam::PRECOMPUTED) return fail("unknown kernel type");
    if (p.gamma < 0) return fail("gamma < 0");
    if (p.degree < 0) return fail("degree of polynomial kernel < 0");
    if (p.epsilon <= 0) return fail("epsilon <= 0");
    const bool uses_c = p.svm_type == SvmParam::C_SVC || p.svm_type == SvmParam::EPSILON_SVR || p.svm_type == SvmParam::NU_SVR;
    const bool uses_nu = p.svm_type == SvmParam::NU_SVC || p.svm_type == SvmParam::ONE_CLASS || p.svm_type == SvmParam::NU_SVR;
    if (uses_c && p.C <= 0) return fail("C <= 0");
    if (uses_nu && (p.nu <= 0 || p.nu > 1)) return fail("nu <= 0 or nu > 1");
    // a class weight of zero makes that class's C zero: its instances belong to neither I_up nor I_low and the
    // working set may not fill (the solver reports that case; rejecting it here gives the clearer message)
    for (int i = 0; i < p.nr_weight; ++i)
        if (p.weight[i] <= 0) return fail("class weight <= 0");
    if (p.svm_type == SvmParam::EPSILON_SVR && p.p < 0) return fail("p < 0");
    if (p.max_mem_size <= 0) return fail("max memory size <= 0");
    if (p.probability != 0 && p.probability != 1) return fail("probability != 0 and probability != 1");
    if (p.probability == 1 && (p.svm_type == SvmParam::ONE_CLASS || p.svm_type == SvmParam::EPSILON_SVR ||
                               p.svm_type == SvmParam::NU_SVR))
        return fail("one-class SVM and SVR probability output not supported yet");
    return true;
}
