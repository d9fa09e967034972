// TEST INFRASTRUCTURE — C entry points over the reference project's own, unmodified CUDA
// kernels. The wrapper translation units include the reference's .cu files from where they
// lie in the reference checkout (nothing is copied); only the built library travels.
// Used by the GPU tests as a second reference and by the bench's reference arm.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
// kernels/skip_layernorm.cu:101-112 launcher, as shipped.
int ref_skip_layernorm(half* in_out, const half* skip, const half* gamma, const half* beta,
                       int num, int size, cudaStream_t stream);
// kernels/linear.cu:54-150 kernels, launched with grid (N/16, T/16) and the row pitch of X
// passed in the kernel's `M` slot (the shipped launcher passes the token count there, which is
// only right when tokens == in_feat).
int ref_tile_spmm(half* Y, const half* X, const int* row_ptr, const int* row_offset,
                  const half* data, int T, int N, int K, const half* bias, int gelu,
                  cudaStream_t stream);
// kernels/linear.cu:18-34 launcher (bias fill + cuBLAS GEMM), as shipped. N must be a multiple of 2.
int ref_row_spmm(half* out, const half* in, const half* weight, const half* bias, int M, int N,
                 int K, cudaStream_t stream);
// kernels/attention.cu:51-120 kernel for one sequence. scale <= 0 selects the shipped
// launcher's own scale, sqrt(1/head_dim); seq_len must be a multiple of 16.
int ref_otf_attention(half* out, const half* Q, const half* K, const half* V, const half* mask,
                      int seq_len, int d_model, int nhead, float scale, cudaStream_t stream);
// kernels/attention.cu:273-350 launcher, as shipped (ignores its stream argument).
int ref_sharedqk_attention(half* out, const half* QK, const half* V, const half* mask,
                           int seq_len, int d_model, int nhead);
// The same kernel on a caller-chosen stream (the shipped launcher always uses the default stream).
int ref_sharedqk_attention_on(half* out, const half* QK, const half* V, const half* mask,
                              int seq_len, int d_model, int nhead, cudaStream_t stream);
// kernels/attention.cu:149-250 kernel for one sequence, launched with the shipped launcher's
// configuration (kernels/attention.cu:252-271: 512 threads, its shared-memory size, scale
// sqrt(1/head_dim)) on `stream`. As shipped the kernel computes the attention and never stores
// it (kernels/attention.cu:242-248): `out` is left untouched. For timing only.
int ref_prune_attention(half* out, const half* Q, const half* K, const half* V,
                        const int* v_col_id, const int* v_head_ptr, int nnz_col_v, const half* mask,
                        int seq_len, int d_model, int nhead, cudaStream_t stream);
// The scores GEMM of Encoder_length::run (encoder/encoder.cu:126-130) for one sequence with Q and K
// as the linears produce them (row pitch d_model, head h in columns h*head_dim..): one
// cublasHgemmStridedBatched over the heads, QK[h][q][k] = scale * Q_h[q] . K_h[k].
int ref_qk_scores(half* QK, const half* Q, const half* K, int seq_len, int d_model, int nhead,
                  cudaStream_t stream);
// One encoder layer over `batch` sequences of `seq_len` tokens in the op order of
// encoder/encoder.cu:20-45, on one stream and without host synchronisation: the six linears
// and both LayerNorms run once over all tokens, attention once per sequence.
// bsr[6] = {Q,K,V,O,FFN1,FFN2}, each {row_ptr,row_offset,data,bias}. buffer: 8*T*d_model halfs.
typedef struct {
    const int* row_ptr;
    const int* row_offset;
    const half* data;
    const half* bias;
} ref_bsr_t;
int ref_encoder_tile_layer(half* out, const half* in, half* buffer, const ref_bsr_t* bsr,
                           const half* ln_gamma0, const half* ln_beta0, const half* ln_gamma1,
                           const half* ln_beta1, const half* mask, int batch, int seq_len,
                           int d_model, int nhead, int d_ff, float scale, cudaStream_t stream);
// Attention-aware pruned layer in the op order of encoder/encoder.cu:65-92: Q and K through the
// tile kernel (bsr[0], bsr[1]), V through the row-pruned launcher (cuBLAS, kernels/linear.cu:18-34)
// from the compact weight [nnz_v x d_model], the shipped pruned-attention kernel once per sequence
// (it stores nothing, so the attention-output buffer keeps whatever it held: timing only), then the
// tile / LayerNorm tail. bsr[2] is unused. buffer: 8*T*d_model halfs.
int ref_encoder_prune_layer(half* out, const half* in, half* buffer, const ref_bsr_t* bsr,
                            const half* v_weight, const half* v_bias, const int* v_row_id,
                            const int* v_head_ptr, int nnz_v, const half* ln_gamma0,
                            const half* ln_beta0, const half* ln_gamma1, const half* ln_beta1,
                            const half* mask, int batch, int seq_len, int d_model, int nhead,
                            int d_ff, cudaStream_t stream);
// Sequence-aware layer in the op order of encoder/encoder.cu:116-149 over packed sequences whose
// lengths (host array) are multiples of 16: linears and LayerNorms once over all tokens; per
// sequence the scores GEMM into `scores` (nhead * max_len^2 halfs, reused) and the shared-QK
// attention kernel with the given mask (max_len x max_len zeros serve every length).
int ref_encoder_length_layer(half* out, const half* in, half* buffer, half* scores,
                             const ref_bsr_t* bsr, const half* ln_gamma0, const half* ln_beta0,
                             const half* ln_gamma1, const half* ln_beta1, const half* mask,
                             const int* seq_lens_host, int batch, int d_model, int nhead, int d_ff,
                             cudaStream_t stream);
#ifdef __cplusplus
}
#endif
