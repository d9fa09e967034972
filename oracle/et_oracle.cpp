// TEST INFRASTRUCTURE — CPU oracle for the E.T. encoder hot path.
//
// Plain C++ fp32 restatement of the arithmetic the reference's CUDA kernels are meant to
// perform. Only the tests, the smoke check and the bench's cpu_baseline / reference arm
// may load this library, and only as the checker or as a timed baseline; the product
// library never links or calls it.
//
// Parity status: the reference ships no expected outputs of any kind (its three
// executables print nothing and check nothing), so this oracle cannot be pinned against
// reference golden vectors. It is pinned instead against outputs of the reference's own
// CUDA kernels run on a B200 (fixtures under tests/golden/, produced by
// tests/golden/make_golden.py) in the `ET_ORC_REF_COMPAT` mode that reproduces the
// reference's base-2 exponent and zero-initialised row max.
//
// Reference files restated here (paths inside the reference project):
//   encoder/encoder.cu:20-45      op order of one post-LN encoder layer
//   kernels/linear.cu:36-48       tanh-GELU
//   kernels/linear.cu:54-101      16x16 tile-BSR linear  Y = X W^T + bias
//   kernels/linear.cu:18-34       row-pruned linear (compact output features)
//   encoder/Linear.cu:74-88       head_ptr of a row-pruned linear (intended CSR prefix)
//   kernels/attention.cu:10-48    row softmax
//   kernels/attention.cu:51-120   on-the-fly attention for one (query block, head)
//   kernels/attention.cu:149-250  attention with column-pruned V (intended scatter)
//   kernels/attention.cu:273-340  mask + softmax + P.V from precomputed scores
//   kernels/skip_layernorm.cu:4-43 residual add + LayerNorm, eps 1e-6, two-pass variance
//   test/tile_mat.cu:5-34, test/row_mat.cu:5-14   pruned-format generators
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- fp16 <-> fp32 (round to nearest even), no hardware half type needed ----
inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t f2h(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((x > 0x7f800000u) ? 0x200u : 0));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);       // rounds to inf
    if (x < 0x33000001u) return (uint16_t)sign;                    // rounds to zero
    int e = (int)(x >> 23) - 127;
    uint32_t m = (x & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t hm = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (hm & 1))) ++hm;
    uint32_t he = (e < -14) ? 0 : (uint32_t)(e + 15);
    // hm carries the implicit bit for normals; adding handles mantissa overflow
    uint32_t out = (e < -14) ? hm : ((he << 10) + (hm - 0x400u));
    return (uint16_t)(sign | out);
}

// ---- counter-free splitmix64 stream: the one generator shared by every seeded structure ----
struct SplitMix {
    uint64_t s;
    explicit SplitMix(uint64_t seed) : s(seed) {}
    uint64_t next() {
        uint64_t z = (s += 0x9e3779b97f4a7c15ull);
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        return z ^ (z >> 31);
    }
    double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
};

template <class T> void shuffle(std::vector<T>& v, SplitMix& rng) {
    for (size_t i = v.size(); i > 1; --i) {
        size_t j = (size_t)(rng.next() % (uint64_t)i);
        std::swap(v[i - 1], v[j]);
    }
}

inline float gelu_tanh(float x) {
    return 0.5f * x * (1.0f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

constexpr int FLAG_REF_COMPAT = 1;  // base-2 exponent, row max initialised to 0

// softmax over `n` entries of `row` (already scaled and masked); entries beyond `valid` are dropped.
inline void softmax_row(float* row, int n, int valid, int flags) {
    const bool compat = flags & FLAG_REF_COMPAT;
    float mx = compat ? 0.0f : -INFINITY;
    for (int i = 0; i < valid; ++i) mx = std::max(mx, row[i]);
    if (!(mx > -INFINITY)) {                       // every key masked: defined as all zeros
        for (int i = 0; i < n; ++i) row[i] = 0.0f;
        return;
    }
    float sum = 0.0f;
    for (int i = 0; i < valid; ++i) {
        float e = compat ? std::exp2(row[i] - mx) : std::exp(row[i] - mx);
        row[i] = e;
        sum += e;
    }
    float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (int i = 0; i < valid; ++i) row[i] *= inv;
    for (int i = valid; i < n; ++i) row[i] = 0.0f;
}

}  // namespace

extern "C" {

int orc_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

float orc_h2f(uint16_t h) { return h2f(h); }
uint16_t orc_f2h(float f) { return f2h(f); }

void orc_round_half(float* x, long n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) x[i] = h2f(f2h(x[i]));
}

// ---------------------------------------------------------------------------------------------
// Pruned-format generators.
// Tile format (test/tile_mat.cu:5-34): W[nrow x ncol] cut into 16x16 tiles; row_ptr has
// nrow/16+1 entries; row_offset[i] is the input-feature offset (a multiple of 16) of kept
// tile i. mode 0 keeps exactly floor(total*(1-sparsity)) tiles drawn by a shuffle and lists a
// block-row's tiles in shuffle order (tile_mat.cu:11-29); mode 1 keeps each tile
// independently with probability 1-sparsity and lists them by ascending offset.
// Returns the kept-tile count, or -1 if `cap` is too small.
// ---------------------------------------------------------------------------------------------
int orc_gen_sparse_tile_mat(int nrow, int ncol, float sparsity, uint64_t seed, int mode,
                            int* row_ptr, int* row_offset, int cap) {
    const int br = nrow / 16, bc = ncol / 16;
    const long total = (long)br * bc;
    SplitMix rng(seed);
    std::vector<std::vector<int>> per_row(br);
    if (mode == 0) {
        const long ntile = (long)((double)total * (1.0 - (double)sparsity));
        std::vector<int> ids(total);
        std::iota(ids.begin(), ids.end(), 0);
        shuffle(ids, rng);
        for (long i = 0; i < ntile; ++i) per_row[ids[i] / bc].push_back((ids[i] % bc) * 16);
    } else {
        const double keep = 1.0 - (double)sparsity;
        for (int r = 0; r < br; ++r)
            for (int c = 0; c < bc; ++c)
                if (rng.uniform() < keep) per_row[r].push_back(c * 16);
    }
    int off = 0;
    row_ptr[0] = 0;
    for (int r = 0; r < br; ++r) {
        if (off + (int)per_row[r].size() > cap) return -1;
        for (int c : per_row[r]) row_offset[off++] = c;
        row_ptr[r + 1] = off;
    }
    return off;
}

// Row format (test/row_mat.cu:5-14): exactly floor(nrow*(1-sparsity)) kept output rows,
// sorted ascending. The draw is repeated until every head keeps at least one row (nhead > 0).
int orc_gen_sparse_row_mat(int nrow, float sparsity, uint64_t seed, int nhead, int* row_id,
                           int cap) {
    const int keep = (int)((double)nrow * (1.0 - (double)sparsity));
    if (keep > cap) return -1;
    SplitMix rng(seed);
    std::vector<int> ids(nrow);
    for (int attempt = 0; attempt < 1000; ++attempt) {
        std::iota(ids.begin(), ids.end(), 0);
        shuffle(ids, rng);
        std::vector<int> kept(ids.begin(), ids.begin() + keep);
        std::sort(kept.begin(), kept.end());
        bool ok = true;
        if (nhead > 0) {
            const int hd = nrow / nhead;
            std::vector<int> cnt(nhead, 0);
            for (int r : kept) cnt[r / hd]++;
            for (int c : cnt) ok = ok && c > 0;
        }
        if (ok) {
            std::copy(kept.begin(), kept.end(), row_id);
            return keep;
        }
    }
    return -2;
}

// head_ptr[h] = number of kept rows with original index < h*head_dim, h = 0..nhead
// (the CSR prefix encoder/Linear.cu:74-88 intends).
void orc_head_ptr(const int* row_id, int n, int nhead, int out_feat, int* head_ptr) {
    const int hd = out_feat / nhead;
    int i = 0;
    for (int h = 0; h <= nhead; ++h) {
        while (i < n && row_id[i] < h * hd) ++i;
        head_ptr[h] = i;
    }
}

// Dense [N x K] view of a tile-BSR weight; data[i*256 + n*16 + k] = W[16r+n, row_offset[i]+k]
// (kernels/linear.cu:76).
void orc_bsr_to_dense(float* W, const int* row_ptr, const int* row_offset, const float* data,
                      int N, int K) {
    std::fill(W, W + (size_t)N * K, 0.0f);
    for (int r = 0; r < N / 16; ++r)
        for (int i = row_ptr[r]; i < row_ptr[r + 1]; ++i)
            for (int n = 0; n < 16; ++n)
                for (int k = 0; k < 16; ++k)
                    W[(size_t)(16 * r + n) * K + row_offset[i] + k] += data[(size_t)i * 256 + n * 16 + k];
}

// ---------------------------------------------------------------------------------------------
// Y[T x N] = X[T x K] . W^T + bias, optional tanh-GELU (kernels/linear.cu:54-150). X pitch K.
// Zero tiles are skipped, as in the reference.
// ---------------------------------------------------------------------------------------------
void orc_tile_linear(float* Y, const float* X, const int* row_ptr, const int* row_offset,
                     const float* data, const float* bias, int T, int N, int K, int gelu) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        const float* x = X + (size_t)t * K;
        float* y = Y + (size_t)t * N;
        for (int r = 0; r < N / 16; ++r) {
            float acc[16];
            for (int n = 0; n < 16; ++n) acc[n] = 0.0f;
            for (int i = row_ptr[r]; i < row_ptr[r + 1]; ++i) {
                const float* w = data + (size_t)i * 256;
                const float* xs = x + row_offset[i];
                for (int n = 0; n < 16; ++n) {
                    float s = 0.0f;
                    for (int k = 0; k < 16; ++k) s += xs[k] * w[n * 16 + k];
                    acc[n] += s;
                }
            }
            for (int n = 0; n < 16; ++n) {
                float v = acc[n] + (bias ? bias[16 * r + n] : 0.0f);
                y[16 * r + n] = gelu ? gelu_tanh(v) : v;
            }
        }
    }
}

// out[T x nkeep] (pitch out_pitch) = in[T x K] . weight[nkeep x K]^T + bias
// (kernels/linear.cu:18-34: bias broadcast, then GEMM with beta = 1).
void orc_row_linear(float* out, const float* in, const float* weight, const float* bias, int T,
                    int nkeep, int K, int out_pitch) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        const float* x = in + (size_t)t * K;
        for (int n = 0; n < nkeep; ++n) {
            const float* w = weight + (size_t)n * K;
            float s = 0.0f;
            for (int k = 0; k < K; ++k) s += x[k] * w[k];
            out[(size_t)t * out_pitch + n] = s + (bias ? bias[n] : 0.0f);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Attention over a batch of packed sequences (kernels/attention.cu:67-119 per sequence).
//   Q, K : [sum(seq_lens) x q_pitch]; V : [sum(seq_lens) x v_pitch]; Z : [sum(seq_lens) x d_model].
//   qk_head_ptr == null: head h of Q/K is columns [h*hd, (h+1)*hd). Otherwise Q/K are compact
//     and head h is columns [qk_head_ptr[h], qk_head_ptr[h+1]) (retained dims shared by Q, K).
//   v_head_ptr == null: dense V as above. Otherwise V is compact; head h owns compact columns
//     [v_head_ptr[h], v_head_ptr[h+1]) and result column j is written to Z column v_col_id[j]
//     (kernels/attention.cu:214-248 as intended); every other Z column of the row is 0.
//   mask: additive [mask_ld x mask_ld] shared by all heads and sequences, or null.
//   valid_lens: keys >= valid_lens[b] are excluded (key padding); null means seq_lens.
//   scale is always 1/sqrt(d_model/nhead) (kernels/attention.cu:126).
// ---------------------------------------------------------------------------------------------
void orc_attention(float* Z, const float* Q, const float* K, const float* V, int q_pitch,
                   int v_pitch, const int* qk_head_ptr, const int* v_col_id,
                   const int* v_head_ptr, const float* mask, int mask_ld, const int* seq_lens,
                   const int* valid_lens, int batch, int d_model, int nhead, int flags) {
    const int hd = d_model / nhead;
    const float scale = 1.0f / std::sqrt((float)hd);
    std::vector<long> start(batch + 1, 0);
    for (int b = 0; b < batch; ++b) start[b + 1] = start[b] + seq_lens[b];
    std::fill(Z, Z + (size_t)start[batch] * d_model, 0.0f);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < nhead; ++h) {
            const int L = seq_lens[b];
            const int valid = valid_lens ? std::min(valid_lens[b], L) : L;
            const int qk0 = qk_head_ptr ? qk_head_ptr[h] : h * hd;
            const int qkw = qk_head_ptr ? qk_head_ptr[h + 1] - qk_head_ptr[h] : hd;
            const int v0 = v_head_ptr ? v_head_ptr[h] : h * hd;
            const int vw = v_head_ptr ? v_head_ptr[h + 1] - v_head_ptr[h] : hd;
            std::vector<float> p(L);
            std::vector<float> o(vw);
            for (int q = 0; q < L; ++q) {
                const float* qr = Q + (size_t)(start[b] + q) * q_pitch + qk0;
                for (int k = 0; k < valid; ++k) {
                    const float* kr = K + (size_t)(start[b] + k) * q_pitch + qk0;
                    float s = 0.0f;
                    for (int d = 0; d < qkw; ++d) s += qr[d] * kr[d];
                    s *= scale;
                    if (mask) s += mask[(size_t)q * mask_ld + k];
                    p[k] = s;
                }
                softmax_row(p.data(), L, valid, flags);
                std::fill(o.begin(), o.end(), 0.0f);
                for (int k = 0; k < valid; ++k) {
                    const float* vr = V + (size_t)(start[b] + k) * v_pitch + v0;
                    const float pk = p[k];
                    for (int d = 0; d < vw; ++d) o[d] += pk * vr[d];
                }
                float* zr = Z + (size_t)(start[b] + q) * d_model;
                for (int d = 0; d < vw; ++d) zr[v_head_ptr ? v_col_id[v0 + d] : v0 + d] = o[d];
            }
        }
    }
}

// Scores S[h][q][k] = scale * Q_h[q] . K_h[k] for one sequence; Q, K pitch d_model
// (what encoder/encoder.cu:126-130 intends to materialise).
void orc_scores(float* S, const float* Q, const float* K, int L, int d_model, int nhead) {
    const int hd = d_model / nhead;
    const float scale = 1.0f / std::sqrt((float)hd);
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < nhead; ++h)
        for (int q = 0; q < L; ++q)
            for (int k = 0; k < L; ++k) {
                float s = 0.0f;
                for (int d = 0; d < hd; ++d)
                    s += Q[(size_t)q * d_model + h * hd + d] * K[(size_t)k * d_model + h * hd + d];
                S[((size_t)h * L + q) * L + k] = s * scale;
            }
}

// In-place masked softmax over scores [nmat][L][L]; the mask [L x L] (nullable) is shared by
// all matrices; keys >= valid are dropped (kernels/attention.cu:297-323 over full rows).
void orc_softmax_mask(float* S, const float* mask, int nmat, int L, int valid, int flags) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < nmat; ++h)
        for (int q = 0; q < L; ++q) {
            float* row = S + ((size_t)h * L + q) * L;
            if (mask)
                for (int k = 0; k < valid; ++k) row[k] += mask[(size_t)q * L + k];
            softmax_row(row, L, valid, flags);
        }
}

// Z = softmax(S + mask) . V per head from precomputed scores (kernels/attention.cu:273-340).
void orc_sharedqk_attention(float* Z, const float* S, const float* V, const float* mask, int L,
                            int d_model, int nhead, int flags) {
    const int hd = d_model / nhead;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < nhead; ++h)
        for (int q = 0; q < L; ++q) {
            std::vector<float> p(L);
            for (int k = 0; k < L; ++k)
                p[k] = S[((size_t)h * L + q) * L + k] + (mask ? mask[(size_t)q * L + k] : 0.0f);
            softmax_row(p.data(), L, L, flags);
            for (int d = 0; d < hd; ++d) {
                float s = 0.0f;
                for (int k = 0; k < L; ++k) s += p[k] * V[(size_t)k * d_model + h * hd + d];
                Z[(size_t)q * d_model + h * hd + d] = s;
            }
        }
}

// in_out <- LayerNorm(in_out + skip) * gamma + beta, rows of `size`
// (kernels/skip_layernorm.cu:19-42: mean, then sum of squared deviations, eps 1e-6).
void orc_skip_layernorm(float* in_out, const float* skip, const float* gamma, const float* beta,
                        int num, int size) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < num; ++r) {
        float* x = in_out + (size_t)r * size;
        const float* s = skip + (size_t)r * size;
        float mean = 0.0f;
        for (int i = 0; i < size; ++i) {
            x[i] += s[i];
            mean += x[i];
        }
        mean /= (float)size;
        float var = 0.0f;
        for (int i = 0; i < size; ++i) var += (x[i] - mean) * (x[i] - mean);
        const float rstd = 1.0f / std::sqrt(var / (float)size + 1e-6f);
        for (int i = 0; i < size; ++i) x[i] = (x[i] - mean) * rstd * gamma[i] + beta[i];
    }
}

}  // extern "C"
