// Host runtime pieces shared by the model layer: verbosity switch, device-memory helpers behind
// SyncArray, the parameter name tables and the two metrics.
#include <thundersvm/thundersvm.h>
#include <thundersvm/syncarray.h>
#include <thundersvm/svmparam.h>
#include <thundersvm/util/metric.h>
#include <cuda_runtime.h>
#include "../common.cuh"

namespace thundersvm {
bool g_verbose = true;
void set_verbose(bool on) { g_verbose = on; }

static void cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return;
    if (e == cudaErrorMemoryAllocation) throw std::bad_alloc();       // reference: util/common.h:33-39
    LOG(FATAL) << what << ": " << cudaGetErrorString(e);
}
// SyncArray memory comes from the library's pool (a model trains one binary problem per class pair, each
// with its own arrays)
void *device_alloc(size_t bytes) {
    void *p = nullptr;
    const tsvm_status s = tsvm::pool_alloc(&p, bytes ? bytes : 1);
    if (s == TSVM_ERR_OOM) throw std::bad_alloc();                    // reference: util/common.h:33-39
    if (s != TSVM_OK) LOG(FATAL) << "device allocation: " << tsvm_last_error();
    return p;
}
void device_free(void *p) { tsvm::pool_free(p); }
static thread_local cudaStream_t tl_stream = nullptr;
cudaStream_t work_stream() { return tl_stream; }
void set_work_stream(cudaStream_t s) { tl_stream = s; }
// Copies are ordered on the calling thread's stream; those that touch host memory return when they are done,
// as cudaMemcpy does.
void copy_to_device(void *dst, const void *src, size_t bytes) {
    cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, tl_stream), "H2D copy");
    cuda_ok(cudaStreamSynchronize(tl_stream), "H2D copy");
}
void copy_to_host(void *dst, const void *src, size_t bytes) {
    cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, tl_stream), "D2H copy");
    cuda_ok(cudaStreamSynchronize(tl_stream), "D2H copy");
}
void copy_on_device(void *dst, const void *src, size_t bytes) {
    cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, tl_stream), "D2D copy");
}
void device_zero(void *p, size_t bytes) { cuda_ok(cudaMemsetAsync(p, 0, bytes, tl_stream), "cudaMemset"); }
std::atomic<size_t> &total_memory_size() {
    static std::atomic<size_t> bytes{0};
    return bytes;
}
}  // namespace thundersvm

const char *SvmParam::kernel_type_name[6] = {"linear", "polynomial", "rbf", "sigmoid", "precomputed", "NULL"};
const char *SvmParam::svm_type_name[6] = {"c_svc", "nu_svc", "one_class", "epsilon_svr", "nu_svr", "NULL"};

string Accuracy::name() { return "Accuracy"; }
float_type Accuracy::score(const vector<float_type> &predict_y, const vector<float_type> &ground_truth_y) {
    size_t hits = 0;
    for (size_t i = 0; i < predict_y.size(); ++i) hits += predict_y[i] == ground_truth_y[i];
    return hits / (float) ground_truth_y.size();
}
string MSE::name() { return "Mean Squared Error"; }
float_type MSE::score(const vector<float_type> &predict_y, const vector<float_type> &ground_truth_y) {
    float_type acc = 0;
    for (size_t i = 0; i < predict_y.size(); ++i) {
        const float_type e = predict_y[i] - ground_truth_y[i];
        acc += e * e;
    }
    return acc / predict_y.size();
}
