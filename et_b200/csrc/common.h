// Shared host-side helpers of the C-ABI layer: status codes, last-error text, argument checks.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
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

}  // namespace et

#define ET_REQUIRE(cond, msg) \
    do {                      \
        if (!(cond)) return et::fail(ET_ERR_INVALID, msg); \
    } while (0)
