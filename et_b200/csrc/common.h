// Shared host-side helpers of the C-ABI layer: status codes, last-error text, argument checks.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include "../../include/et_b200.h"

namespace et {

void set_error(const char* fmt, ...);

inline int fail(int code, const char* what) {
    set_error("%s", what);
    return code;
}
inline int cuda_status(cudaError_t e, const char* where) {
    if (e == cudaSuccess) return ET_OK;
    set_error("%s: %s", where, cudaGetErrorString(e));
    return ET_ERR_CUDA;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int sm_count() {
    static int n = [] {
        int dev = 0, v = 148;
        if (cudaGetDevice(&dev) == cudaSuccess)
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v;
    }();
    return n;
}

// Runs `f` once per device (function attributes such as the shared-memory opt-in belong to a device's context,
// not to the process) and returns its result on every later call from that device.
struct PerDeviceOnce {
    std::mutex mu;
    bool done[64] = {};
    cudaError_t err[64] = {};
    template <typename F>
    cudaError_t run(F&& f) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lk(mu);
        if (!done[dev]) {
            err[dev] = f();
            done[dev] = true;
        }
        return err[dev];
    }
};

// Programmatic dependent launch: the kernel may be scheduled while its predecessor in the stream is still
// running; it must execute pdl_wait() before it touches anything the predecessor writes or reads.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
// Blocks until every kernel this one depends on has completed and its writes are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream start its own prologue.
__device__ __forceinline__ void pdl_launch_dependents() {
#ifndef ET_NO_EARLY_PDL
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
#endif

}  // namespace et

#define ET_REQUIRE(cond, msg) \
    do {                      \
        if (!(cond)) return et::fail(ET_ERR_INVALID, msg); \
    } while (0)
