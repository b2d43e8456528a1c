// thundersvm-predict: prediction CLI (reference: src/thundersvm/thundersvm-predict.cpp:18-106).
#include <thundersvm/svm_interface_api.h>
#include <thundersvm/thundersvm.h>
#include <exception>
#include <new>

int main(int argc, char **argv) {
    try {
        thundersvm_predict(argc, argv);
    } catch (std::bad_alloc &) {
        std::cerr << "out of memory, you may try \"-m memory size\" to constrain memory usage" << std::endl;
        return EXIT_FAILURE;
    } catch (std::exception const &x) {
        std::cerr << x.what() << std::endl;
        return EXIT_FAILURE;
    } catch (...) {
        std::cerr << "unknown error" << std::endl;
        return EXIT_FAILURE;
    }
    return 0;
}
