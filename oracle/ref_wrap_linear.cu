// TEST INFRASTRUCTURE — see ref_wrap.h.
#include <cuda_fp16.h>
#include <kernels/kernels.h>
;
#include <kernels/linear.cu>
#include "ref_wrap.h"

extern "C" int ref_tile_spmm(half* Y, const half* X, const int* row_ptr, const int* row_offset,
                             const half* data, int T, int N, int K, const half* bias, int gelu,
                             cudaStream_t stream) {
    if (T % 16 || N % 16 || K % 16) return 1;
    dim3 grid(N / 16, T / 16);
    if (gelu)
        __kernel_blk_mmul_blk_bias_smem_cta_skew_gelu<128>
            <<<grid, 128, 0, stream>>>(Y, X, row_ptr, row_offset, data, K, N, bias);
    else
        __kernel_blk_mmul_blk_bias_smem_cta_skew<128>
            <<<grid, 128, 0, stream>>>(Y, X, row_ptr, row_offset, data, K, N, bias);
    return (int)cudaGetLastError();
}

static cublasHandle_t ref_handle() {
    static cublasHandle_t handle = nullptr;
    if (!handle && cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) handle = nullptr;
    return handle;
}

extern "C" int ref_qk_scores(half* QK, const half* Q, const half* K, int seq_len, int d_model,
                             int nhead, cudaStream_t stream) {
    cublasHandle_t handle = ref_handle();
    if (!handle) return 2;
    cublasSetStream(handle, stream);
    const int head_dim = d_model / nhead;
    const half scale = __float2half(1.0f / sqrtf((float)head_dim)), beta = __float2half(0.0f);
    // column-major view: C[key][query] with leading dimension seq_len is QK[query][key] row-major
    const cublasStatus_t st = cublasHgemmStridedBatched(
        handle, CUBLAS_OP_T, CUBLAS_OP_N, seq_len, seq_len, head_dim, &scale, K, d_model, head_dim,
        Q, d_model, head_dim, &beta, QK, seq_len, (long long)seq_len * seq_len, nhead);
    return st == CUBLAS_STATUS_SUCCESS ? 0 : 3;
}

extern "C" int ref_row_spmm(half* out, const half* in, const half* weight, const half* bias,
                            int M, int N, int K, cudaStream_t stream) {
    cublasHandle_t handle = ref_handle();
    if (!handle) return 2;
    cublasSetStream(handle, stream);
    row_spmm_add_bias_kernelLauncher(out, in, weight, bias, M, N, K, handle,
                                     CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    return (int)cudaGetLastError();
}
