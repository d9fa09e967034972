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
