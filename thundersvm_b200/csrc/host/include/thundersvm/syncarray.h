// SyncArray<T>: a host vector with a lazily allocated device mirror, the argument type of the
// reference's solver / kernel-matrix API (include/thundersvm/syncarray.h:16-108,
// src/thundersvm/syncmem.cpp:58-134). The side written last is the valid one; asking for the other
// side copies the whole buffer. set_host_data / set_device_data alias foreign memory without owning
// it. A process-wide byte counter feeds SvmModel::get_working_set_size as in the reference.
#ifndef THUNDERSVM_SYNCARRAY_H
#define THUNDERSVM_SYNCARRAY_H
#include <atomic>
#include <cuda_runtime.h>
#include "thundersvm.h"
#include <cstring>
#include <new>

namespace thundersvm {
void *device_alloc(size_t bytes);                 // throws std::bad_alloc when the device is out of memory
void device_free(void *p);
void copy_to_device(void *dst, const void *src, size_t bytes);
void copy_to_host(void *dst, const void *src, size_t bytes);
void copy_on_device(void *dst, const void *src, size_t bytes);
void device_zero(void *p, size_t bytes);
std::atomic<size_t> &total_memory_size();
// The CUDA stream this host thread's copies and library calls go to (nullptr: the default stream). SVC::train
// gives each of its worker threads a stream of its own.
cudaStream_t work_stream();
void set_work_stream(cudaStream_t s);
}  // namespace thundersvm

template <typename T>
class SyncArray {
public:
    explicit SyncArray(size_t count) { resize(count); }
    SyncArray() {}
    ~SyncArray() { release(); }
    SyncArray(const SyncArray &) = delete;
    SyncArray &operator=(const SyncArray &) = delete;

    size_t size() const { return size_; }
    size_t mem_size() const { return size_ * sizeof(T); }

    void resize(size_t count) {
        release();
        size_ = count;
        host_.assign(count, T());
        thundersvm::total_memory_size() += mem_size();
        head_ = HOST;
    }

    const T *host_data() const { to_host(); return hptr(); }
    T *host_data() { to_host(); head_ = HOST; return hptr(); }
    const T *device_data() const { to_device(); return dev_; }
    T *device_data() { to_device(); head_ = DEVICE; return dev_; }

    void to_host() const {
        if (head_ == DEVICE && dev_) { thundersvm::copy_to_host(hptr(), dev_, mem_size()); head_ = BOTH; }
    }
    void to_device() const {
        if (!dev_ && size_) {
            dev_ = static_cast<T *>(thundersvm::device_alloc(mem_size()));
            own_dev_ = true;
            if (head_ == DEVICE) thundersvm::device_zero(dev_, mem_size());
        }
        if (head_ == HOST && size_) { thundersvm::copy_to_device(dev_, hptr(), mem_size()); head_ = BOTH; }
    }

    void copy_from(const T *source, size_t count) {
        CHECK_LE(count, size_) << "copy_from: source larger than the array";
        std::memcpy(host_data(), source, sizeof(T) * count);
    }
    void copy_from(const SyncArray<T> &source) {
        CHECK_EQ(size_, source.size()) << "copy_from: size mismatch";
        if (source.head_ == DEVICE && source.dev_) thundersvm::copy_on_device(device_data(), source.dev_, mem_size());
        else std::memcpy(host_data(), source.hptr(), mem_size());
    }
    void mem_set(const T &value) {
        T *h = host_data();
        for (size_t i = 0; i < size_; ++i) h[i] = value;
    }
    // alias foreign buffers (no ownership)
    void set_host_data(T *p) { ext_host_ = p; head_ = HOST; }
    void set_device_data(T *p) {
        if (own_dev_ && dev_) thundersvm::device_free(dev_);
        dev_ = p; own_dev_ = false; head_ = DEVICE;
    }

private:
    enum Head { HOST, DEVICE, BOTH };
    T *hptr() const { return ext_host_ ? ext_host_ : const_cast<T *>(host_.data()); }
    void release() {
        if (own_dev_ && dev_) thundersvm::device_free(dev_);
        dev_ = nullptr; own_dev_ = false; ext_host_ = nullptr;
        if (size_) thundersvm::total_memory_size() -= mem_size();
        size_ = 0;
    }
    size_t size_ = 0;
    mutable vector<T> host_;
    T *ext_host_ = nullptr;
    mutable T *dev_ = nullptr;
    mutable bool own_dev_ = false;
    mutable Head head_ = HOST;
};
#endif
