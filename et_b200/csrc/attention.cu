// On-the-fly multi-head attention  Z_h = softmax(scale * Q_h K_h^T + mask) V_h  over a batch of packed,
// variable-length sequences; the S x S score matrix never goes to HBM.
// Replaces kernels/attention.cu of the reference: the on-the-fly kernel (:51-134), the variant with
// column-pruned V (:149-271, including the scatter of the result that the shipped kernel computes but
// never stores) and the variant that reads precomputed scores (:273-350).
//
// One kernel covers all variants through a per-head column window on each operand:
//   dense      : head h of Q/K/V is columns [h*hd, (h+1)*hd)
//   pruned V   : V is compact [tokens x nnz]; head h owns compact columns [v_head_ptr[h], v_head_ptr[h+1]),
//                result column j goes to Z column v_col_id[j], all other Z columns of the head are 0
//   pruned Q/K : Q and K compact with the same retained dims per head (qk_head_ptr)
//   scores     : Q K^T is read from HBM ([nhead][L][L], already scaled) instead of computed
// Length-driven tiling: the grid is sized by the number of 64-query blocks actually present
// (sum over sequences of ceil(len/64)); a CTA walks only ceil(valid/64) key blocks; lengths need not be
// multiples of 16. fp32 softmax statistics, true row max, ex2 with log2(e) folded into the scale;
// a fully masked row gives zeros.
//
// Tensor path: warp-level mma.sync m16n8k16 with ldmatrix-fed fragments (flash-style online softmax,
// P stays in registers). Widths per head up to 64 are supported (zero-padded in shared memory).
#include <mutex>
#include "attention.h"
#include "common.h"

namespace et {

namespace {

constexpr int kBQ = 64;    // queries per CTA (16 per warp)
constexpr int kBK = 64;    // keys per block
constexpr int kD = 64;     // padded per-head width
constexpr int kPitch = kD + 8;  // shared-memory row pitch in halfs (144 B: conflict-free ldmatrix)

struct AttnParams {
    const half* Q; const half* K; const half* V; half* Z;
    const half* mask; const half* scores;
    int q_pitch, v_pitch, z_pitch, mask_ld;
    const int* cu_seqlens; const int* valid_lens;
    int batch, uniform_len, nhead, head_dim;
    const int* qk_head_ptr; const int* v_head_ptr; const int* v_col_id;
    float scale_log2;
};

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Copies rows [row0, row0+64) x columns [col0, col0+width) of a [*, pitch] matrix into a zero-padded
// 64 x 64 shared tile; rows >= row_end are zero.
__device__ __forceinline__ void load_tile(half* dst, const half* __restrict__ src, long row0, long row_end,
                                          int pitch, int col0, int width, int tid) {
    const bool vec = ((pitch & 7) == 0) && ((col0 & 7) == 0) && ((width & 7) == 0) &&
                     ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    if (vec) {
        for (int i = tid; i < kBK * (kD / 8); i += 128) {
            const int r = i >> 3, c = (i & 7) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row0 + r < row_end && c < width)
                v = __ldg(reinterpret_cast<const uint4*>(src + (row0 + r) * pitch + col0 + c));
            *reinterpret_cast<uint4*>(dst + r * kPitch + c) = v;
        }
    } else {
        for (int i = tid; i < kBK * kD; i += 128) {
            const int r = i >> 6, c = i & 63;
            half v = __float2half(0.f);
            if (row0 + r < row_end && c < width) v = src[(row0 + r) * pitch + col0 + c];
            dst[r * kPitch + c] = v;
        }
    }
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = pred ? 16 : 0;   // 0: nothing is read, the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// load_tile with 16-byte asynchronous copies where the operand allows it (aligned window), else synchronous.
__device__ __forceinline__ void load_tile_async(half* dst, const half* __restrict__ src, long row0, long row_end,
                                                int pitch, int col0, int width, int tid) {
    const bool vec = ((pitch & 7) == 0) && ((col0 & 7) == 0) && ((width & 7) == 0) &&
                     ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    if (!vec) {
        load_tile(dst, src, row0, row_end, pitch, col0, width, tid);
        return;
    }
    for (int i = tid; i < kBK * (kD / 8); i += 128) {
        const int r = i >> 3, c = (i & 7) * 8;
        const bool in = row0 + r < row_end && c < width;
        cp_async16(dst + r * kPitch + c, in ? src + (row0 + r) * pitch + col0 + c : src, in);
    }
}

__global__ void __launch_bounds__(128) attention_kernel(const AttnParams p) {
    __shared__ __align__(16) half sQ[kBQ * kPitch];
    __shared__ __align__(16) half sKb[2][kBK * kPitch];   // two stages: block kb+1 streams in while kb is used
    __shared__ __align__(16) half sVb[2][kBK * kPitch];
    __shared__ int s_seq[3];  // sequence index, first token, query offset inside the sequence

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y;

    // ---- which (sequence, query block) is this CTA?
    if (tid == 0) {
        int b = -1, tok0 = 0, q0 = 0;
        int blk = blockIdx.x;
        if (p.cu_seqlens) {
            for (int i = 0; i < p.batch; ++i) {
                const int L = p.cu_seqlens[i + 1] - p.cu_seqlens[i];
                const int nb = (L + kBQ - 1) / kBQ;
                if (blk < nb) { b = i; tok0 = p.cu_seqlens[i]; q0 = blk * kBQ; break; }
                blk -= nb;
            }
        } else {
            const int nb = (p.uniform_len + kBQ - 1) / kBQ;
            if (blk < nb * p.batch) { b = blk / nb; tok0 = b * p.uniform_len; q0 = (blk % nb) * kBQ; }
        }
        s_seq[0] = b; s_seq[1] = tok0; s_seq[2] = q0;
    }
    __syncthreads();
    const int b = s_seq[0];
    if (b < 0) return;
    const long tok0 = s_seq[1];
    const int q0 = s_seq[2];
    const int L = p.cu_seqlens ? p.cu_seqlens[b + 1] - p.cu_seqlens[b] : p.uniform_len;
    int valid = p.valid_lens ? p.valid_lens[b] : L;
    valid = valid < L ? valid : L;

    const int hd = p.head_dim;
    const int qk0 = p.qk_head_ptr ? p.qk_head_ptr[h] : h * hd;
    const int qkw = p.qk_head_ptr ? p.qk_head_ptr[h + 1] - qk0 : hd;
    const int v0 = p.v_head_ptr ? p.v_head_ptr[h] : h * hd;
    const int vw = p.v_head_ptr ? p.v_head_ptr[h + 1] - v0 : hd;
    const int ksteps = (qkw + 15) >> 4;       // k16 steps of Q K^T that hold data
    const int vtiles = (vw + 7) >> 3;         // n8 tiles of P V that hold data

    const int nkb = (valid + kBK - 1) / kBK;
    // Q and the first key/value block are requested together; later blocks are requested one ahead.
    if (nkb > 0) {
        if (!p.scores) {
            load_tile_async(sQ, p.Q, tok0 + q0, tok0 + L, p.q_pitch, qk0, qkw, tid);
            load_tile_async(sKb[0], p.K, tok0, tok0 + valid, p.q_pitch, qk0, qkw, tid);
        }
        load_tile_async(sVb[0], p.V, tok0, tok0 + valid, p.v_pitch, v0, vw, tid);
        cp_async_commit();
    }
    // pruned V: the head's whole Z window starts as zero, retained columns are scattered over it later
    if (p.v_head_ptr) {
        for (int i = tid; i < kBQ * hd; i += 128) {
            const int r = i / hd, c = i % hd;
            if (q0 + r < L) p.Z[(tok0 + q0 + r) * p.z_pitch + h * hd + c] = __float2half(0.f);
        }
    }

    uint32_t qf[4][4];
    float o[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g+8 of this warp's 16
    const int qr0 = q0 + warp * 16 + g, qr1 = qr0 + 8;          // query index inside the sequence

    for (int kb = 0; kb < nkb; ++kb) {
        const int k0 = kb * kBK;
        const half* sK = sKb[kb & 1];
        const half* sV = sVb[kb & 1];
        if (kb + 1 < nkb) {
            if (!p.scores)
                load_tile_async(sKb[(kb + 1) & 1], p.K, tok0 + k0 + kBK, tok0 + valid, p.q_pitch, qk0, qkw, tid);
            load_tile_async(sVb[(kb + 1) & 1], p.V, tok0 + k0 + kBK, tok0 + valid, p.v_pitch, v0, vw, tid);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kb == 0 && !p.scores) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                        sQ + (warp * 16 + (lane & 15)) * kPitch + ks * 16 + (lane >> 4) * 8);
        }

        float s[8][4];
        if (!p.scores) {
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                if (ks < ksteps) {
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) {
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4(b0, b1, b2, b3,
                                sK + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kPitch + ks * 16 + ((lane >> 3) & 1) * 8);
                        mma16816(s[2 * jp], qf[ks], b0, b1);
                        mma16816(s[2 * jp + 1], qf[ks], b2, b3);
                    }
                }
            }
        } else {
            const half* S = p.scores + ((size_t)b * p.nhead + h) * (size_t)L * L;  // one sequence per matrix set
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kc = k0 + j * 8 + 2 * t;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int qr = r ? qr1 : qr0;
                    float a = 0.f, c = 0.f;
                    if (qr < L) {
                        if (kc < L) a = __half2float(S[(size_t)qr * L + kc]);
                        if (kc + 1 < L) c = __half2float(S[(size_t)qr * L + kc + 1]);
                    }
                    s[j][2 * r] = a; s[j][2 * r + 1] = c;
                }
            }
        }
        // scale (log2 domain), additive mask, key validity
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int kc = k0 + j * 8 + 2 * t;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = kc + (e & 1);
                const int qr = (e & 2) ? qr1 : qr0;
                float v = s[j][e] * p.scale_log2;
                if (p.mask && qr < L && k < valid)
                    v += __half2float(__ldg(p.mask + (size_t)qr * p.mask_ld + k)) * 1.4426950408889634f;
                if (k >= valid) v = -INFINITY;
                s[j][e] = v;
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float sh0 = (mn0 == -INFINITY) ? 0.f : mn0, sh1 = (mn1 == -INFINITY) ? 0.f : mn1;
        const float c0 = exp2f(m0 - sh0), c1 = exp2f(m1 - sh1);   // m = -inf gives 0
        m0 = mn0; m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = exp2f(s[j][0] - sh0); s[j][1] = exp2f(s[j][1] - sh0);
            s[j][2] = exp2f(s[j][2] - sh1); s[j][3] = exp2f(s[j][3] - sh1);
            rs0 += s[j][0] + s[j][1];
            rs1 += s[j][2] + s[j][3];
        }
        l0 = l0 * c0 + rs0; l1 = l1 * c1 + rs1;
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack_half2(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_half2(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                if (2 * jp < vtiles) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(b0, b1, b2, b3,
                              sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kPitch + jp * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * jp], a, b0, b1);
                    mma16816(o[2 * jp + 1], a, b2, b3);
                }
            }
        }
        __syncthreads();   // this stage is overwritten by the request issued in the next iteration
    }
    // ---- finalize: divide by the row sum (per-thread partial sums are combined across the quad)
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    __syncthreads();   // zero-fill of the pruned window (above) is ordered before the scatter
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = j * 8 + 2 * t;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int qr = r ? qr1 : qr0;
            if (qr >= L) continue;
            const float x = o[j][2 * r] * (r ? inv1 : inv0), y = o[j][2 * r + 1] * (r ? inv1 : inv0);
            half* zrow = p.Z + (tok0 + qr) * p.z_pitch;
            if (p.v_head_ptr) {
                if (c < vw) zrow[p.v_col_id[v0 + c]] = __float2half_rn(x);
                if (c + 1 < vw) zrow[p.v_col_id[v0 + c + 1]] = __float2half_rn(y);
            } else if (c + 1 < vw) {
                *reinterpret_cast<half2*>(zrow + v0 + c) = __floats2half2_rn(x, y);
            } else if (c < vw) {
                zrow[v0 + c] = __float2half_rn(x);
            }
        }
    }
}

// Scores S[h][q][k] = scale * Q_h[q] . K_h[k] for `batch` equal-length sequences, written to HBM as
// [batch][nhead][L][L] fp16 (what the reference materialises with a strided-batched GEMM,
// encoder/encoder.cu:126-130). grid = (q blocks, k blocks, batch*nhead).
__global__ void __launch_bounds__(128) qk_scores_kernel(half* __restrict__ S, const half* __restrict__ Q,
                                                        const half* __restrict__ K, int L, int pitch,
                                                        int nhead, int hd, float scale) {
    __shared__ __align__(16) half sQ[kBQ * kPitch];
    __shared__ __align__(16) half sK[kBK * kPitch];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z / nhead, h = blockIdx.z % nhead;
    const int q0 = blockIdx.x * kBQ, k0 = blockIdx.y * kBK;
    const long tok0 = (long)b * L;
    load_tile(sQ, Q, tok0 + q0, tok0 + L, pitch, h * hd, hd, tid);
    load_tile(sK, K, tok0 + k0, tok0 + L, pitch, h * hd, hd, tid);
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const int ksteps = (hd + 15) >> 4;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        if (ks < ksteps) {
            uint32_t a[4];
            ldsm_x4(a[0], a[1], a[2], a[3], sQ + (warp * 16 + (lane & 15)) * kPitch + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3,
                        sK + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kPitch + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816(s[2 * jp], a, b0, b1);
                mma16816(s[2 * jp + 1], a, b2, b3);
            }
        }
    }
    half* out = S + (size_t)blockIdx.z * L * L;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int kc = k0 + j * 8 + 2 * t;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int qr = q0 + warp * 16 + g + 8 * r;
            if (qr >= L) continue;
            if (kc < L) out[(size_t)qr * L + kc] = __float2half_rn(s[j][2 * r] * scale);
            if (kc + 1 < L) out[(size_t)qr * L + kc + 1] = __float2half_rn(s[j][2 * r + 1] * scale);
        }
    }
}

}  // namespace

int qk_scores_launch(half* S, const half* Q, const half* K, int batch, int L, int d_model, int nhead,
                     cudaStream_t st, int pitch) {
    if (pitch <= 0) pitch = d_model;
    if (!S || !Q || !K) return fail(ET_ERR_INVALID, "qk scores: null pointer");
    if (batch < 0 || L < 0 || nhead <= 0 || d_model <= 0 || d_model % nhead) return fail(ET_ERR_INVALID, "qk scores: bad dimensions");
    const int hd = d_model / nhead;
    if (hd > kD) return fail(ET_ERR_UNSUPPORTED, "qk scores: head_dim above 64 is not supported");
    if (batch == 0 || L == 0) return ET_OK;
    if ((long)batch * nhead > 65535) return fail(ET_ERR_UNSUPPORTED, "qk scores: batch*nhead above 65535");
    dim3 grid((L + kBQ - 1) / kBQ, (L + kBK - 1) / kBK, batch * nhead);
    return cuda_status(launch_pdl(qk_scores_kernel, grid, dim3(128), 0, st, S, Q, K, L, pitch, nhead, hd,
                                  1.0f / sqrtf((float)hd)),
                       "qk scores launch");
}

int attention_launch(half* Z, const half* Q, const half* K, const half* V, const half* scores,
                     int q_pitch, int v_pitch, const int* qk_head_ptr, const int* v_col_id,
                     const int* v_head_ptr, const half* mask, int mask_ld, const int* cu_seqlens,
                     const int* valid_lens, int batch, int uniform_len, int total_tokens, int d_model,
                     int nhead, cudaStream_t st, int max_len) {
    if (!Z || !V || (!scores && (!Q || !K))) return fail(ET_ERR_INVALID, "attention: null pointer");
    if (batch < 0 || nhead <= 0 || d_model <= 0 || d_model % nhead) return fail(ET_ERR_INVALID, "attention: bad dimensions");
    const int hd = d_model / nhead;
    if (hd > kD) return fail(ET_ERR_UNSUPPORTED, "attention: head_dim above 64 is not supported");
    if (hd % 2 || (d_model % 2)) return fail(ET_ERR_INVALID, "attention: head_dim must be even");
    if ((v_head_ptr == nullptr) != (v_col_id == nullptr)) return fail(ET_ERR_INVALID, "attention: v_head_ptr and v_col_id go together");
    if (mask && mask_ld <= 0) return fail(ET_ERR_INVALID, "attention: mask without leading dimension");
    if (!cu_seqlens && uniform_len <= 0 && batch > 0) return fail(ET_ERR_INVALID, "attention: no lengths given");
    if (batch == 0 || total_tokens == 0) return ET_OK;
    if (scores && cu_seqlens) return fail(ET_ERR_UNSUPPORTED, "attention: precomputed scores need equal-length sequences");
    if (!scores && !qk_head_ptr && !v_head_ptr) {
        // dense case: tensor-core (tcgen05) kernel when the shape is in its range
        const int ml = cu_seqlens ? max_len : uniform_len;
        const int rc = attention_tc_launch(Z, Q, K, V, q_pitch, v_pitch, mask, mask_ld, cu_seqlens, valid_lens, batch,
                                           uniform_len, total_tokens, ml, d_model, nhead, st);
        if (rc != ET_ERR_UNSUPPORTED) return rc;
    }
    AttnParams p;
    p.Q = Q; p.K = K; p.V = V; p.Z = Z; p.mask = mask; p.scores = scores;
    p.q_pitch = q_pitch; p.v_pitch = v_pitch; p.z_pitch = d_model; p.mask_ld = mask_ld;
    p.cu_seqlens = cu_seqlens; p.valid_lens = valid_lens; p.batch = batch; p.uniform_len = uniform_len;
    p.nhead = nhead; p.head_dim = hd; p.qk_head_ptr = qk_head_ptr; p.v_head_ptr = v_head_ptr; p.v_col_id = v_col_id;
    p.scale_log2 = scores ? 1.4426950408889634f : 1.4426950408889634f / sqrtf((float)hd);
    const int nblk = cu_seqlens ? (total_tokens + kBQ - 1) / kBQ + batch
                                : batch * ((uniform_len + kBQ - 1) / kBQ);
    return cuda_status(launch_pdl(attention_kernel, dim3(nblk, nhead), dim3(128), 0, st, p), "attention launch");
}


// ------------------------------------------------------------------------------------------------
// Attention through materialised scores for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a layer: code that
// runs inside a real-time serving loop with a fixed memory plan, a plugin loaded into a process whose
// allocator owns the whole device, or a caller that is between cudaStreamBeginCapture and
// cudaStreamEndCapture for unrelated work on another stream. For them the score matrices
// [nhead][seq_len][seq_len] live in the array below, which is part of the library image: every GPU that
// loads the library holds these 8 MiB until the process exits.
//
// The array is shared by all calls on a device and keeps the contents of the previous call. Nothing
// has to be cleared: the score kernel writes every element that the attention kernel later reads.
// Two calls that overlap on the GPU (different streams, or different host threads) race on it;
// serialise them on one stream.
constexpr size_t kStaticScoreHalfs = (size_t)16 * 512 * 512;   // e.g. 16 heads x 512 x 512
static __device__ __align__(256) half g_static_scores[kStaticScoreHalfs];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
half* g_static_ptr[kMaxDevices] = {nullptr};
}  // namespace

// In host code `g_static_scores` is only a handle for the runtime, not a device address; the address a
// kernel can use is obtained once per device, with that device current.
static int static_scores_address(half** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e, "static scores: cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(ET_ERR_UNSUPPORTED, "static scores: device ordinal above 63");
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scores);
        if (e != cudaSuccess) return cuda_status(e, "static scores: cudaGetSymbolAddress");
        g_static_ptr[dev] = static_cast<half*>(p);
    }
    *out = g_static_ptr[dev];
    return ET_OK;
}

int attention_static_scores(half* Z, const half* Q, const half* K, const half* V, const half* mask, int seq_len,
                            int d_model, int nhead, cudaStream_t st) {
    if (seq_len < 0 || nhead <= 0 || d_model <= 0) return fail(ET_ERR_INVALID, "static-score attention: bad dimensions");
    if ((size_t)nhead * seq_len * seq_len > kStaticScoreHalfs)
        return fail(ET_ERR_UNSUPPORTED,
                    "static-score attention: nhead*seq_len*seq_len exceeds the built-in score buffer (16*512*512 elements)");
    half* scores = nullptr;
    int rc = static_scores_address(&scores);
    if (rc) return rc;
    if ((rc = qk_scores_launch(scores, Q, K, 1, seq_len, d_model, nhead, st))) return rc;
    return attention_launch(Z, nullptr, nullptr, V, scores, d_model, d_model, nullptr, nullptr, nullptr, mask, seq_len,
                            nullptr, nullptr, 1, seq_len, seq_len, d_model, nhead, st);
}

}  // namespace et
