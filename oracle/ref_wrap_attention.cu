// TEST INFRASTRUCTURE — see ref_wrap.h. kernels/attention.cu does not include kernels.h.
#include <kernels/attention.cu>
#include "ref_wrap.h"

extern "C" int ref_otf_attention(half* out, const half* Q, const half* K, const half* V,
                                 const half* mask, int seq_len, int d_model, int nhead,
                                 float scale, cudaStream_t stream) {
    if (seq_len % 16 || d_model % nhead) return 1;
    const int head_dim = d_model / nhead;
    if (head_dim % 16) return 1;
    const half hscale = __float2half(scale > 0.f ? scale : sqrtf(1.0f / head_dim));
    constexpr int num_thd = 256;
    const size_t smem = sizeof(half) * (16 * (head_dim + FP16_skew) + 16 * (seq_len + FP16_skew));
    if (smem > 48 * 1024) return 1;
    __kernel_multi_head_full_skew_warpSFM<num_thd>
        <<<dim3(seq_len / 16, nhead), num_thd, smem, stream>>>(Q, K, V, out, d_model, seq_len,
                                                               head_dim, hscale, mask);
    return (int)cudaGetLastError();
}

extern "C" int ref_sharedqk_attention(half* out, const half* QK, const half* V, const half* mask,
                                      int seq_len, int d_model, int nhead) {
    if (seq_len % 16 || sizeof(half) * 16 * (seq_len + 16) > 48 * 1024) return 1;
    sharedQK_attention_kernelLauncher(out, const_cast<half*>(QK), const_cast<half*>(V),
                                      const_cast<half*>(mask), seq_len, d_model, nhead, nullptr);
    return (int)cudaGetLastError();
}

extern "C" int ref_sharedqk_attention_on(half* out, const half* QK, const half* V, const half* mask,
                                         int seq_len, int d_model, int nhead, cudaStream_t stream) {
    if (seq_len % 16 || sizeof(half) * 16 * (seq_len + 16) > 48 * 1024) return 1;
    constexpr int num_thd = 256;   // kernels/attention.cu:345
    __kernel_multi_head_sharedQK<num_thd>
        <<<dim3(seq_len / 16, nhead), num_thd, sizeof(half) * 16 * (seq_len + FP16_skew), stream>>>(
            QK, V, out, d_model, seq_len, d_model / nhead, mask);
    return (int)cudaGetLastError();
}

extern "C" int ref_prune_attention(half* out, const half* Q, const half* K, const half* V,
                                   const int* v_col_id, const int* v_head_ptr, int nnz_col_v,
                                   const half* mask, int seq_len, int d_model, int nhead,
                                   cudaStream_t stream) {
    if (seq_len % 16 || d_model % nhead || !mask) return 1;
    const int head_dim = d_model / nhead;
    if (head_dim % 16) return 1;
    constexpr int num_thd = 512;   // kernels/attention.cu:266
    const size_t temp_row = 16 * (seq_len + FP16_skew) * sizeof(half);
    const size_t temp_Q = 16 * (head_dim + FP16_skew) * sizeof(half);
    const size_t temp_blk = 16 * ((num_thd / 2) + FP16_skew) * sizeof(half);
    const size_t temp_id = 16 * (num_thd / 32) * sizeof(int);
    const size_t smem = temp_row + (temp_Q > temp_blk + temp_id ? temp_Q : temp_blk + temp_id);
    if (smem > 48 * 1024) return 1;
    const half scale = __float2half(sqrtf(1.0f / head_dim));
    __kernel_multi_head_prune<num_thd><<<dim3(seq_len / 16, nhead), num_thd, smem, stream>>>(
        Q, K, V, out, d_model, seq_len, head_dim, scale, nhead, v_col_id, v_head_ptr, nnz_col_v,
        mask);
    return (int)cudaGetLastError();
}
