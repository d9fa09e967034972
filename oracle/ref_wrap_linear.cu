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

extern "C" int ref_row_spmm(half* out, const half* in, const half* weight, const half* bias,
                            int M, int N, int K, cudaStream_t stream) {
    static cublasHandle_t handle = nullptr;
    if (!handle && cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 2;
    cublasSetStream(handle, stream);
    row_spmm_add_bias_kernelLauncher(out, in, weight, bias, M, N, K, handle,
                                     CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    return (int)cudaGetLastError();
}
