// TEST INFRASTRUCTURE — see ref_wrap.h. Composition of the reference's kernels into one
// encoder layer over a batch, in the op order of encoder/encoder.cu:20-45.
#include "ref_wrap.h"

extern "C" int ref_encoder_tile_layer(half* out, const half* in, half* buffer,
                                      const ref_bsr_t* bsr, const half* ln_gamma0,
                                      const half* ln_beta0, const half* ln_gamma1,
                                      const half* ln_beta1, const half* mask, int batch,
                                      int seq_len, int d_model, int nhead, int d_ff, float scale,
                                      cudaStream_t stream) {
    const int T = batch * seq_len;
    const size_t td = (size_t)T * d_model;
    half* q = buffer;
    half* k = buffer + td;
    half* v = buffer + 2 * td;
    half* z = buffer + 3 * td;
    half* f = buffer + 4 * td;  // T x d_ff (d_ff <= 4*d_model)
    int rc = 0;
    auto lin = [&](half* y, const half* x, int i, int N, int K, int gelu) {
        rc |= ref_tile_spmm(y, x, bsr[i].row_ptr, bsr[i].row_offset, bsr[i].data, T, N, K,
                            bsr[i].bias, gelu, stream);
    };
    lin(q, in, 0, d_model, d_model, 0);
    lin(k, in, 1, d_model, d_model, 0);
    lin(v, in, 2, d_model, d_model, 0);
    for (int b = 0; b < batch; ++b) {
        const size_t o = (size_t)b * seq_len * d_model;
        rc |= ref_otf_attention(z + o, q + o, k + o, v + o, mask, seq_len, d_model, nhead, scale,
                                stream);
    }
    lin(q, z, 3, d_model, d_model, 0);
    rc |= ref_skip_layernorm(q, in, ln_gamma0, ln_beta0, T, d_model, stream);
    lin(f, q, 4, d_ff, d_model, 1);
    lin(out, f, 5, d_model, d_ff, 0);
    rc |= ref_skip_layernorm(out, q, ln_gamma1, ln_beta1, T, d_model, stream);
    return rc;
}

// Tail shared by the three layer kinds: output projection, LayerNorm, FFN, LayerNorm
// (encoder/encoder.cu:34-44, :80-91, :137-148).
static int ref_layer_tail(half* out, const half* in, half* q, half* z, half* f, const ref_bsr_t* bsr,
                          const half* g0, const half* b0, const half* g1, const half* b1, int T,
                          int d_model, int d_ff, cudaStream_t stream) {
    int rc = 0;
    rc |= ref_tile_spmm(q, z, bsr[3].row_ptr, bsr[3].row_offset, bsr[3].data, T, d_model, d_model, bsr[3].bias, 0, stream);
    rc |= ref_skip_layernorm(q, in, g0, b0, T, d_model, stream);
    rc |= ref_tile_spmm(f, q, bsr[4].row_ptr, bsr[4].row_offset, bsr[4].data, T, d_ff, d_model, bsr[4].bias, 1, stream);
    rc |= ref_tile_spmm(out, f, bsr[5].row_ptr, bsr[5].row_offset, bsr[5].data, T, d_model, d_ff, bsr[5].bias, 0, stream);
    rc |= ref_skip_layernorm(out, q, g1, b1, T, d_model, stream);
    return rc;
}

extern "C" int ref_encoder_prune_layer(half* out, const half* in, half* buffer, const ref_bsr_t* bsr,
                                       const half* v_weight, const half* v_bias, const int* v_row_id,
                                       const int* v_head_ptr, int nnz_v, const half* ln_gamma0,
                                       const half* ln_beta0, const half* ln_gamma1,
                                       const half* ln_beta1, const half* mask, int batch, int seq_len,
                                       int d_model, int nhead, int d_ff, cudaStream_t stream) {
    const int T = batch * seq_len;
    const size_t td = (size_t)T * d_model;
    half* q = buffer;
    half* k = buffer + td;
    half* v = buffer + 2 * td;   // T x nnz_v, compact
    half* z = buffer + 3 * td;
    half* f = buffer + 4 * td;
    int rc = 0;
    rc |= ref_tile_spmm(q, in, bsr[0].row_ptr, bsr[0].row_offset, bsr[0].data, T, d_model, d_model, bsr[0].bias, 0, stream);
    rc |= ref_tile_spmm(k, in, bsr[1].row_ptr, bsr[1].row_offset, bsr[1].data, T, d_model, d_model, bsr[1].bias, 0, stream);
    rc |= ref_row_spmm(v, in, v_weight, v_bias, T, nnz_v, d_model, stream);
    for (int b = 0; b < batch; ++b) {
        const size_t o = (size_t)b * seq_len * d_model, ov = (size_t)b * seq_len * nnz_v;
        rc |= ref_prune_attention(z + o, q + o, k + o, v + ov, v_row_id, v_head_ptr, nnz_v, mask, seq_len,
                                  d_model, nhead, stream);
    }
    rc |= ref_layer_tail(out, in, q, z, f, bsr, ln_gamma0, ln_beta0, ln_gamma1, ln_beta1, T, d_model, d_ff, stream);
    return rc;
}

extern "C" int ref_encoder_length_layer(half* out, const half* in, half* buffer, half* scores,
                                        const ref_bsr_t* bsr, const half* ln_gamma0,
                                        const half* ln_beta0, const half* ln_gamma1,
                                        const half* ln_beta1, const half* mask,
                                        const int* seq_lens_host, int batch, int d_model, int nhead,
                                        int d_ff, cudaStream_t stream) {
    int T = 0;
    for (int b = 0; b < batch; ++b) {
        if (seq_lens_host[b] <= 0 || seq_lens_host[b] % 16) return 1;
        T += seq_lens_host[b];
    }
    const size_t td = (size_t)T * d_model;
    half* q = buffer;
    half* k = buffer + td;
    half* v = buffer + 2 * td;
    half* z = buffer + 3 * td;
    half* f = buffer + 4 * td;
    int rc = 0;
    rc |= ref_tile_spmm(q, in, bsr[0].row_ptr, bsr[0].row_offset, bsr[0].data, T, d_model, d_model, bsr[0].bias, 0, stream);
    rc |= ref_tile_spmm(k, in, bsr[1].row_ptr, bsr[1].row_offset, bsr[1].data, T, d_model, d_model, bsr[1].bias, 0, stream);
    rc |= ref_tile_spmm(v, in, bsr[2].row_ptr, bsr[2].row_offset, bsr[2].data, T, d_model, d_model, bsr[2].bias, 0, stream);
    size_t o = 0;
    for (int b = 0; b < batch; ++b) {
        const int L = seq_lens_host[b];
        rc |= ref_qk_scores(scores, q + o, k + o, L, d_model, nhead, stream);
        rc |= ref_sharedqk_attention_on(z + o, scores, v + o, mask, L, d_model, nhead, stream);
        o += (size_t)L * d_model;
    }
    rc |= ref_layer_tail(out, in, q, z, f, bsr, ln_gamma0, ln_beta0, ln_gamma1, ln_beta1, T, d_model, d_ff, stream);
    return rc;
}
