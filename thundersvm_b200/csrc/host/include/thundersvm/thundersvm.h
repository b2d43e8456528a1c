// Host-side mirror of the reference's basic types (include/thundersvm/thundersvm.h:16-22):
// float_type = double for alpha / f / rho / coefficients / decision values, kernel_type = float
// for feature and kernel values. Logging is a small stream class instead of easylogging++:
// LOG(INFO|WARNING|ERROR) print when verbose, LOG(FATAL) always prints and aborts, CHECK* abort.
#ifndef THUNDERSVM_THUNDERSVM_H
#define THUNDERSVM_THUNDERSVM_H
#include <cmath>
#include <cstdlib>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

using std::string;
using std::vector;
typedef double float_type;
typedef float kernel_type;

namespace thundersvm {
extern bool g_verbose;                 // toggled by -q / the `verbose` arguments of the C API
void set_verbose(bool on);

class LogLine {
public:
    LogLine(const char *level, bool fatal) : fatal_(fatal), on_(fatal || g_verbose) { if (on_) ss_ << level << " "; }
    ~LogLine() {
        if (on_) (fatal_ ? std::cerr : std::cout) << ss_.str() << std::endl;
        if (fatal_) std::abort();
    }
    template <typename T>
    LogLine &operator<<(const T &v) { if (on_) ss_ << v; return *this; }
private:
    bool fatal_, on_;
    std::ostringstream ss_;
};
}  // namespace thundersvm

#define TSVM_LOG_INFO thundersvm::LogLine("INFO", false)
#define TSVM_LOG_WARNING thundersvm::LogLine("WARNING", false)
#define TSVM_LOG_ERROR thundersvm::LogLine("ERROR", false)
#define TSVM_LOG_FATAL thundersvm::LogLine("FATAL", true)
#define LOG(level) TSVM_LOG_##level
#define CHECK(cond) if (!(cond)) LOG(FATAL) << "Check failed: " #cond " "
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_GE(a, b) CHECK((a) >= (b))
#define CHECK_LE(a, b) CHECK((a) <= (b))
#define CHECK_NOTNULL(p) CHECK((p) != nullptr)
#endif
