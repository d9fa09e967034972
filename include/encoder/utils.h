// cudaChk and Weight<T> with the members the reference's callers use (encoder/utils.h:4-43).
#pragma once
#include <cuda_runtime.h>
#include <cassert>
#include <cstdio>
#include <cstdlib>

#define cudaChk(call) ::et_shim::cuda_check((call), __FILE__, __LINE__)

namespace et_shim {

inline void cuda_check(cudaError_t status, const char* file, int line) {
    if (status == cudaSuccess) return;
    std::fprintf(stderr, "CUDA Error: %s %s %d\n", cudaGetErrorString(status), file, line);
    std::exit(1);
}
}  // namespace et_shim

// Owning device array. Constructed from a host pointer it uploads `size` elements; move-only.
template <typename T>
class Weight {
    T* dev_ = nullptr;
    int count_ = 0;

  public:
    Weight() = default;
    explicit Weight(int size) : count_(size) { alloc(size); }
    Weight(T* host, int size) : count_(size) {
        alloc(size);
        set(host);
    }
    Weight(const Weight&) = delete;
    Weight& operator=(const Weight&) = delete;
    Weight(Weight&& other) noexcept : dev_(other.dev_), count_(other.count_) { other.dev_ = nullptr; }
    ~Weight() {
        if (dev_) cudaChk(cudaFree(dev_));
    }
    T* get() { return dev_; }
    const T* get() const { return dev_; }
    int size() const { return count_; }
    void alloc(int size) { cudaChk(cudaMalloc(&dev_, sizeof(T) * (size > 0 ? size : 1))); }
    void set(T* host) { cudaChk(cudaMemcpy(dev_, host, sizeof(T) * count_, cudaMemcpyHostToDevice)); }
};
