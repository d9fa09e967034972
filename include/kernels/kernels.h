// The seven operator launchers of the reference (kernels/kernels.h:3-34), same names and argument order,
// as inline forwards to the C ABI of libet_b200.so. A failure prints et_last_error() and aborts, which is
// what the reference's own error handling (assert / exit) amounts to; callers that want status codes use
// include/et_b200.h directly.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include "../et_b200.h"

// cuBLAS is not used by this library. The two cuBLAS types in the reference's signature are kept as opaque
// stand-ins unless <cublas_v2.h> was included first, so callers need neither the header nor the library.
#if defined(__has_include)
#if __has_include(<cublas_v2.h>)
#include <cublas_v2.h>   // types only: no cuBLAS function is called, nothing to link
#endif
#endif
#if !defined(CUBLAS_V2_H_) && !defined(ET_SHIM_NO_CUBLAS_STANDINS)
struct cublasContext;
typedef struct cublasContext* cublasHandle_t;
typedef int cublasGemmAlgo_t;
#ifndef CUBLAS_GEMM_DEFAULT_TENSOR_OP
#define CUBLAS_GEMM_DEFAULT_TENSOR_OP 99
#endif
#endif

namespace et_shim {
// A null stream means the default stream of the CALLER's translation unit: the per-thread one when the caller is
// compiled with --default-stream per-thread (as the reference is, CMakeLists.txt:13), else the legacy one. The
// library itself is compiled without that flag, so the choice has to be made here, in the caller's code.
inline cudaStream_t stream_of(cudaStream_t s) {
#ifdef CUDA_API_PER_THREAD_DEFAULT_STREAM
    return s ? s : cudaStreamPerThread;
#else
    return s;
#endif
}
inline void require_ok(int status, const char* what) {
    if (status != ET_OK) {
        std::fprintf(stderr, "%s failed (%d): %s\n", what, status, et_last_error());
        std::abort();
    }
}
}  // namespace et_shim

inline void skip_layernorm_kernelLauncher(half* in_out, const half* skip, const half* gamma, const half* beta,
                                          int num, int size, cudaStream_t stream) {
    et_shim::require_ok(et_skip_layernorm(in_out, skip, gamma, beta, num, size, et_shim::stream_of(stream)), "skip_layernorm");
}

// The handle's stream is not consulted (no cuBLAS here): the work goes to the default stream, which is the
// per-thread stream under --default-stream per-thread as in the reference build.
inline void row_spmm_add_bias_kernelLauncher(half* out, const half* in, const half* weight, const half* bias, int M,
                                             int N, int K, cublasHandle_t /*handle*/, cublasGemmAlgo_t /*algo*/) {
    et_shim::require_ok(et_row_spmm_bias(out, in, weight, bias, M, N, K, et_shim::stream_of(nullptr)), "row_spmm_add_bias");
}

// With an explicit K (row pitch of X = in_feat).
inline void tile_spmm_add_bias_kernelLauncher(half* Y, half* X, int* W_row_ptr, int* W_row_offset, half* W_data,
                                              int M, int N, int K, half* bias, cudaStream_t stream) {
    et_shim::require_ok(et_tile_spmm_bias(Y, X, W_row_ptr, W_row_offset, W_data, M, N, K, bias, 0, et_shim::stream_of(stream)),
                        "tile_spmm_add_bias");
}
inline void tile_spmm_add_bias_gelu_kernelLauncher(half* Y, half* X, int* W_row_ptr, int* W_row_offset,
                                                   half* W_data, int M, int N, int K, half* bias,
                                                   cudaStream_t stream) {
    et_shim::require_ok(et_tile_spmm_bias(Y, X, W_row_ptr, W_row_offset, W_data, M, N, K, bias, 1, et_shim::stream_of(stream)),
                        "tile_spmm_add_bias_gelu");
}
// The reference's 9-argument form has no K and reads X with pitch M; it is only meaningful when the token
// count equals in_feat, which is what these overloads assume.
inline void tile_spmm_add_bias_kernelLauncher(half* Y, half* X, int* W_row_ptr, int* W_row_offset, half* W_data,
                                              int M, int N, half* bias, cudaStream_t stream) {
    tile_spmm_add_bias_kernelLauncher(Y, X, W_row_ptr, W_row_offset, W_data, M, N, M, bias, stream);
}
inline void tile_spmm_add_bias_gelu_kernelLauncher(half* Y, half* X, int* W_row_ptr, int* W_row_offset,
                                                   half* W_data, int M, int N, half* bias, cudaStream_t stream) {
    tile_spmm_add_bias_gelu_kernelLauncher(Y, X, W_row_ptr, W_row_offset, W_data, M, N, M, bias, stream);
}

inline void OTF_attention_kernelLauncher(half* out, half* Q, half* K, half* V, half* mask, int seq_len, int d_model,
                                         int nhead, cudaStream_t stream) {
    et_shim::require_ok(et_attention_otf(out, Q, K, V, mask, seq_len, d_model, nhead, et_shim::stream_of(stream)), "OTF_attention");
}

inline void Prune_attention_kernelLauncher(half* out, half* Q, half* K, half* V, int* v_col_id, int* v_head_ptr,
                                           int nnz_col_v, half* mask, int seq_len, int d_model, int nhead,
                                           cudaStream_t stream = nullptr) {
    et_shim::require_ok(et_attention_prune(out, Q, K, V, v_col_id, v_head_ptr, nnz_col_v, mask, seq_len, d_model,
                                           nhead, et_shim::stream_of(stream)),
                        "Prune_attention");
}

inline void sharedQK_attention_kernelLauncher(half* out, half* QK, half* V, half* mask, int seq_len, int d_model,
                                              int nhead, cudaStream_t stream = nullptr) {
    et_shim::require_ok(et_attention_sharedqk(out, QK, V, mask, seq_len, d_model, nhead, et_shim::stream_of(stream)),
                        "sharedQK_attention");
}
