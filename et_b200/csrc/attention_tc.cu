// On-the-fly attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA) for the dense case with
// head_dim 64: the fast path behind et_attention_otf /
// et_attention_batch (the mma.sync kernel in attention.cu covers every other variant).
// Replaces kernels/attention.cu:51-134 of the reference for that case.
//
// A CTA owns 128 queries of one head of one sequence, one TMEM lane and one thread per query:
//   S_j = Q K_j^T      SS UMMA 128x64x16 (x4), Q and the 64-key block K_j in shared memory (TMA, 128-byte
//                      swizzle), S_j accumulated in fp16 (as the reference's kernels accumulate their scores) in 64
//                      TMEM columns
//   softmax            four warps, one thread per query row, one pass per block: the row's 64 scores come out of
//                      tensor memory two to a register (tcgen05.ld.pack::16b); row maximum, scale and reference point
//                      (log2 domain) and the exponentials in packed fp16 arithmetic, no conversion; additive mask
//                      and key validity in fp32 where a block needs them; if the maximum has grown by more than 2^8
//                      the reference point moves and O is rescaled in place; P_j = 2^(s - reference) as packed fp16
//                      over the first 32 score columns (tcgen05.st), row sum in fp32. No exchange between threads,
//                      no second pass
//   O += P_j V_j       TS UMMA 128x64x16 (x4): A = P_j read from tensor memory, B = V_j in shared memory as loaded
//                      (rows = keys), used as an MN-major operand; Q K_{j+1}^T is issued right behind it into the
//                      columns that hold P_j (tcgen05 operations execute in issue order)
//   epilogue           O / row sum -> fp16 -> global, rows beyond the sequence are not written
// The S x S matrix never leaves the SM. K_j / V_j stream through a two-stage ring. A CTA needs 48 KB of shared
// memory, 128 TMEM columns and 160 threads, so four CTAs share an SM: while one CTA's softmax runs, the UMMAs,
// loads and hand-overs of the other three are in flight. Every mbarrier wait is bounded; a wait that gives up
// sets the error word and the CTA leaves through the common exit, freeing its tensor memory.
#include <mutex>
#include "attention.h"
#include "common.h"
#include "ptx.cuh"
#include "tmap.h"

namespace et {

namespace {

// 64 keys per block and one thread per query row, four CTAs per SM. Measured at 256 x 512 tokens, 16 heads, with fp32
// scores: 731 us; 128 keys and two CTAs per SM 812 us; two threads per row and three CTAs per SM 801 us; the earlier
// two-pass form with 128 keys, two threads per row and two CTAs per SM 767 us. Sixteen resident softmax warps with
// the shortest hand-overs between them win. With fp16 scores (below) 597 us.
constexpr int kBQ = 128, kBK = 64, kHD = 64;
constexpr int kNCh = kBK / 32;            // 32-column chunks of a score row
// The kernel is a template on how Q K^T is accumulated. fp16, as the reference's kernels do (kernels/attention.cu:82:
// c_t<half>), is the default: the scores come out of tensor memory already packed two to a register, the common pass
// needs no fp32 -> fp16 conversion and half the registers. Its error grows with the size of the scores (one fp16
// rounding of each 16-term partial sum): against exact arithmetic 2e-3 in the worst element for |q.k| up to 50, 1.4e-2
// up to 165, 3e-2 up to 390. fp32 (attention_tc_set_scores_fp32) keeps 2e-3 throughout and takes ~1.5 times as long.
constexpr int kTile = kBQ * kHD * 2;      // 16 KB: the 128 x 64 fp16 Q tile
constexpr int kKVTile = kBK * kHD * 2;    // one key block of K or V
constexpr int kSoftmaxWarps = 4;          // one thread per query row
constexpr int kThreads = 32 * (kSoftmaxWarps + 1);   // + 1 warp whose lane 0 issues TMA and UMMA
constexpr int kCtasPerSm = 4;
constexpr int kTmemCols = 128;            // S 64 (P overlays its first 32 columns) | O 64: four CTAs share an SM's tensor memory
constexpr uint32_t kPCol = 0, kOCol = kBK;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.f;       // log2 units by which a row maximum must grow before O is rescaled

struct TcParams {
    half* Z;
    const half* mask;
    const int* cu_seqlens;
    const int* valid_lens;
    int z_pitch, mask_ld, batch, uniform_len;
    float scale_log2;
    int* err;
    long long* prof;   // ET_ATTN_PROFILE builds: clock64 stamps of CTA (0,0)
};

#ifdef ET_ATTN_PROFILE
#define AT_STAMP(slot) do { if (p.prof && blockIdx.x == 0 && blockIdx.y == 0) p.prof[(slot)] = clock64(); } while (0)
#else
#define AT_STAMP(slot) do { } while (0)
#endif

struct TcShared {
    uint64_t q_full, k_full[2], v_full[2];   // K/V blocks stream through a two-stage ring
    uint64_t s_ready, p_ready, pv_done, o_done;
    uint32_t tmem_base;
    int seq[3];
    volatile int abort;
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for two fp16 values at once (one special-function op); P is stored in fp16 anyway.
__device__ __forceinline__ uint32_t ex2_h2(uint32_t x) {
    uint32_t y;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Sum of 32 packed fp16 values (each <= 1): two levels of packed adds (partial sums <= 4), then fp32. The row sum
// is thereby the sum of exactly the fp16 P values that are multiplied with V.
__device__ __forceinline__ float sum_packed(const uint32_t (&pk)[16]) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const half2* h2 = reinterpret_cast<const half2*>(pk) + 4 * i;
        const float2 f = __half22float2(__hadd2(__hadd2(h2[0], h2[1]), __hadd2(h2[2], h2[3])));
        s += f.x + f.y;
    }
    return s;
}

// 32 additive mask values of one query row (keys k0..k0+31), times log2(e); zero where there is no mask row.
__device__ __forceinline__ void load_mask32(float (&mk)[32], const half* mrow, int k0, int limit, bool vec) {
    if (!mrow) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mk[i] = 0.f;
        return;
    }
    if (vec && k0 + 32 <= limit) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(mrow + k0) + c);
            const half2* h2 = reinterpret_cast<const half2*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h2[i]);
                mk[c * 8 + 2 * i] = f.x * kLog2e;
                mk[c * 8 + 2 * i + 1] = f.y * kLog2e;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) mk[i] = (k0 + i < limit) ? __half2float(__ldg(mrow + k0 + i)) * kLog2e : 0.f;
    }
}

template <bool kScoresF16>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                  const __grid_constant__ CUtensorMap tmK,
                                                                  const __grid_constant__ CUtensorMap tmV,
                                                                  const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = smem + kTile;          // 2 stages
    uint8_t* sV = sK + 2 * kKVTile;      // 2 stages
    TcShared* sh = reinterpret_cast<TcShared*>(sV + 2 * kKVTile);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    if (tid == 0) AT_STAMP(0);
    pdl_launch_dependents();

    // The warp that issues the copies sets up the barriers, finds the CTA's work item and starts the first loads
    // (Q, K_0, V_0, K_1, V_1) before anything CTA-wide happens: they are in flight during the tensor-memory
    // allocation and the rendezvous. Q/K/V come from DRAM, and a wave's CTAs all start together.
    if (warp == kSoftmaxWarps) {
        if (lane == 0) {
            mbar_init(&sh->q_full, 1);
            for (int j = 0; j < 2; ++j) { mbar_init(&sh->k_full[j], 1); mbar_init(&sh->v_full[j], 1); }
            mbar_init(&sh->s_ready, 1);
            mbar_init(&sh->p_ready, kSoftmaxWarps);   // one arrive per softmax warp
            mbar_init(&sh->pv_done, 1);
            mbar_init(&sh->o_done, 1);
            sh->abort = 0;
            fence_mbar_init();
            prefetch_tmap(&tmQ);
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
        }
        pdl_wait();   // lengths and activations come from the preceding kernels
        int b = -1, tok0 = 0, q0 = 0, len = 0;
        if (p.cu_seqlens) {
            // 32 sequences per round: each lane takes one, a prefix sum of their query-block counts locates the block
            int blk = blockIdx.x;
            for (int base = 0; base < p.batch && b < 0; base += 32) {
                const int i = base + lane;
                const int t0 = i < p.batch ? p.cu_seqlens[i] : 0;
                const int Li = i < p.batch ? p.cu_seqlens[i + 1] - t0 : 0;
                const int nbi = (Li + kBQ - 1) / kBQ;
                int incl = nbi;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                const unsigned hit = __ballot_sync(0xffffffffu, blk < incl);
                if (hit) {
                    const int src = __ffs(hit) - 1;
                    const int excl = __shfl_sync(0xffffffffu, incl - nbi, src);
                    b = base + src;
                    tok0 = __shfl_sync(0xffffffffu, t0, src);
                    len = __shfl_sync(0xffffffffu, Li, src);
                    q0 = (blk - excl) * kBQ;
                } else {
                    blk -= __shfl_sync(0xffffffffu, incl, 31);
                }
            }
        } else {
            const int nb = (p.uniform_len + kBQ - 1) / kBQ;
            const int blk = blockIdx.x;
            if (blk < nb * p.batch) { b = blk / nb; tok0 = b * p.uniform_len; q0 = (blk % nb) * kBQ; len = p.uniform_len; }
        }
        int nvalid = 0;
        if (b >= 0) nvalid = p.valid_lens ? min(p.valid_lens[b], len) : len;
        if (lane == 0) {
            sh->seq[0] = b; sh->seq[1] = tok0; sh->seq[2] = q0;
            if (b >= 0 && nvalid > 0) {
                mbar_expect_tx(&sh->q_full, kTile);
                tma_load_2d(sQ, &tmQ, h * kHD, tok0 + q0, &sh->q_full);
                mbar_expect_tx(&sh->k_full[0], kKVTile);
                tma_load_2d(sK, &tmK, h * kHD, tok0, &sh->k_full[0]);
                mbar_expect_tx(&sh->v_full[0], kKVTile);
                tma_load_2d(sV, &tmV, h * kHD, tok0, &sh->v_full[0]);
                if (nvalid > kBK) {
                    mbar_expect_tx(&sh->k_full[1], kKVTile);
                    tma_load_2d(sK + kKVTile, &tmK, h * kHD, tok0 + kBK, &sh->k_full[1]);
                    mbar_expect_tx(&sh->v_full[1], kKVTile);
                    tma_load_2d(sV + kKVTile, &tmV, h * kHD, tok0 + kBK, &sh->v_full[1]);
                }
            }
        }
        __syncwarp();
        tmem_alloc(&sh->tmem_base, kTmemCols);
        tmem_relinquish();
    } else {
        pdl_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    if (tid == 0) AT_STAMP(1);
    const int b = sh->seq[0], tok0 = sh->seq[1], q0 = sh->seq[2];
    int nkb = 0, L = 0, valid = 0;
    if (b >= 0) {
        L = p.cu_seqlens ? p.cu_seqlens[b + 1] - p.cu_seqlens[b] : p.uniform_len;
        valid = p.valid_lens ? min(p.valid_lens[b], L) : L;
        nkb = (valid + kBK - 1) / kBK;
    }

    if (b >= 0 && nkb > 0) {
        if (warp == kSoftmaxWarps) {
            // ---- the issuing warp stays converged: every lane waits on the barriers, one elected lane issues the copies
            // and the UMMAs (tcgen05 instructions issued from a divergent branch are slower)
            auto load_k = [&](int j) {
                const int st = j & 1;
                mbar_expect_tx(&sh->k_full[st], kKVTile);
                tma_load_2d(sK + (size_t)st * kKVTile, &tmK, h * kHD, tok0 + j * kBK, &sh->k_full[st]);
            };
            auto load_v = [&](int j) {
                const int st = j & 1;
                mbar_expect_tx(&sh->v_full[st], kKVTile);
                tma_load_2d(sV + (size_t)st * kKVTile, &tmV, h * kHD, tok0 + j * kBK, &sh->v_full[st]);
            };
            // (Q and the first two K/V blocks were requested before the CTA-wide set-up)
            const uint32_t idesc_qk = make_idesc_f16(128, kBK, false, false, kScoresF16);
            const uint32_t idesc_pv = make_idesc_f16(128, 64, false, true);   // V is an MN-major B operand
            const uint32_t qa = smem_u32(sQ);
            auto issue_qk = [&](int j) {   // S = Q K_j^T into the S columns
                const uint32_t ka = smem_u32(sK + (size_t)(j & 1) * kKVTile);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_f16(tmem, make_smem_desc(qa + ks * 32, 16, 1024, 2), make_smem_desc(ka + ks * 32, 16, 1024, 2),
                             idesc_qk, ks > 0);
                umma_commit(&sh->s_ready);
            };
            if (lane == 0) AT_STAMP(10);
            bool ok = mbar_wait(&sh->q_full, 0) && mbar_wait(&sh->k_full[0], 0);
            if (lane == 0) AT_STAMP(11);
            if (ok) {
                tc_fence_after();
                if (elect_one()) issue_qk(0);
                if (lane == 0) AT_STAMP(13);
            }
            for (int j = 0; j < nkb && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                if (sh->abort) { ok = false; break; }
                // O += P_j V_j once the softmax warps have written P_j (and rescaled O)
                ok = mbar_wait(&sh->p_ready, (uint32_t)j & 1u) && mbar_wait(&sh->v_full[st], ph);
                if (!ok) break;
                if (lane == 0) AT_STAMP(14 + 2 * j);
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t va = smem_u32(sV + (size_t)st * kKVTile);
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks)   // P of keys 16ks..16ks+15: 8 packed columns
                        umma_f16_ts(tmem + kOCol, tmem + kPCol + (uint32_t)(ks * 8), make_smem_desc(va + ks * 2048, 0, 1024, 2),
                                    idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&sh->pv_done);
                }
                if (lane == 0) AT_STAMP(15 + 2 * j);
                if (j + 1 < nkb) {
                    // S_{j+1} right behind it, into the columns that hold P_j: tcgen05 operations execute in issue
                    // order, so Q K_{j+1}^T cannot overwrite P_j before P_j V_j has read it
                    ok = mbar_wait(&sh->k_full[(j + 1) & 1], (uint32_t)((j + 1) >> 1) & 1u);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        issue_qk(j + 1);
                        if (j + 2 < nkb) load_k(j + 2);   // K_j's stage: Q K_j^T completed before the softmax of block j began
                    }
                    if (j + 2 < nkb) {
                        // V_j's stage is free once P_j V_j has completed
                        ok = mbar_wait(&sh->pv_done, (uint32_t)j & 1u);
                        if (!ok) break;
                        if (elect_one()) load_v(j + 2);
                    }
                }
            }
            if (elect_one()) {
                umma_commit(&sh->o_done);
                if (!ok) {
                    atomicExch(p.err, 21);
                    sh->abort = 1;
                }
            }
            __syncwarp();
        } else {
            // ---- softmax warps: one thread per query row (TMEM lane) and key block
            const int quarter = warp & 3;
            const int row = quarter * 32 + lane;
            const int qr = q0 + row;                       // query index inside the sequence
            const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
            const bool has_mask = p.mask != nullptr;   // uniform: the masked code path is separate from the plain one
            const half* mrow = (has_mask && qr < L) ? p.mask + (size_t)qr * p.mask_ld : nullptr;
            const bool mask_vec = has_mask && (p.mask_ld & 7) == 0 && (reinterpret_cast<uintptr_t>(p.mask) & 15) == 0;
            const uint32_t s_addr = tmem + lane_base;           // this row's scores of a block
            const uint32_t p_addr = tmem + lane_base + kPCol;   // its P values as packed fp16 (over the first half of the score columns)
            const uint32_t o_addr = tmem + lane_base + kOCol;   // its 64 output columns
            float m_run = -INFINITY, l_run = 0.f;   // running maximum and running sum of the row
            bool ok = true;
            for (int j = 0; j < nkb; ++j) {
                const bool got = !sh->abort && mbar_wait(&sh->s_ready, (uint32_t)j & 1u);   // every lane waits: no exchange
                if (!got) {
                    ok = false;
                    sh->abort = 1;
                    break;
                }
                if (tid == 0) AT_STAMP(30 + 4 * (j & 3));
                tc_fence_after();
                const int k0 = j * kBK;
                const bool plain = !has_mask && k0 + kBK <= valid;   // uniform: no per-key validity selects needed

                // The row's 64 scores of this block. S_j could only be computed after P_{j-1} V_{j-1} (issue order), so
                // O and the P columns are free to be written from here on.
                uint32_t rp[32];        // fp16 scores: the row's 64 scores, two to a register
                uint32_t rf[kNCh][32];  // fp32 scores
                if constexpr (kScoresF16) {
                    tmem_ld32_pack16(s_addr, rp);
                } else {
#pragma unroll
                    for (int c = 0; c < kNCh; ++c) tmem_ld32(s_addr + c * 32, rf[c]);
                }
                tmem_ld_wait();
                // scores 2i and 2i+1 of chunk c as fp32
                auto score2 = [&](int c, int i) -> float2 {
                    if constexpr (kScoresF16) return __half22float2(*reinterpret_cast<const half2*>(&rp[c * 16 + i]));
                    else return make_float2(__uint_as_float(rf[c][2 * i]), __uint_as_float(rf[c][2 * i + 1]));
                };
                // The general pass (additive mask, keys beyond the valid length): the scaled, masked scores (log2 domain)
                // of one 32-column chunk in fp32. It is evaluated twice per block, for the maximum and for P, so that
                // only the packed scores stay in registers in between.
                auto general_chunk = [&](int c, float (&v)[32]) {
                    const int kc = k0 + c * 32;
                    if (has_mask) {
                        float mk[32];
                        load_mask32(mk, mrow, kc, valid, mask_vec);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 f = score2(c, i);
                            v[2 * i] = (kc + 2 * i < valid) ? fmaf(f.x, p.scale_log2, mk[2 * i]) : -INFINITY;
                            v[2 * i + 1] = (kc + 2 * i + 1 < valid) ? fmaf(f.y, p.scale_log2, mk[2 * i + 1]) : -INFINITY;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 f = score2(c, i);
                            v[2 * i] = (kc + 2 * i < valid) ? f.x * p.scale_log2 : -INFINITY;
                            v[2 * i + 1] = (kc + 2 * i + 1 < valid) ? f.y * p.scale_log2 : -INFINITY;
                        }
                    }
                };
                float bmax = -INFINITY;
                if (plain && kScoresF16) {
                    half2 mx0 = *reinterpret_cast<const half2*>(&rp[0]), mx1 = *reinterpret_cast<const half2*>(&rp[1]);
#pragma unroll
                    for (int i = 2; i < 32; i += 2) {
                        mx0 = __hmax2(mx0, *reinterpret_cast<const half2*>(&rp[i]));
                        mx1 = __hmax2(mx1, *reinterpret_cast<const half2*>(&rp[i + 1]));
                    }
                    const float2 f = __half22float2(__hmax2(mx0, mx1));
                    bmax = fmaxf(f.x, f.y) * p.scale_log2;   // the scale is positive: scale the maximum once
                } else if (plain) {
                    float raw[kNCh];
#pragma unroll
                    for (int c = 0; c < kNCh; ++c) raw[c] = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
#pragma unroll
                        for (int c = 0; c < kNCh; ++c) raw[c] = fmaxf(raw[c], __uint_as_float(rf[c][i]));
                    }
#pragma unroll
                    for (int c = 0; c < kNCh; ++c) bmax = fmaxf(bmax, raw[c]);
                    bmax *= p.scale_log2;
                } else {
#pragma unroll
                    for (int c = 0; c < kNCh; ++c) {
                        float v[32];
                        general_chunk(c, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) bmax = fmaxf(bmax, v[i]);
                    }
                }
                // The reference point is kept representable in fp16 (the packed pass subtracts it in fp16), within range.
                if (bmax > -INFINITY) bmax = __half2float(__float2half_rn(fminf(fmaxf(bmax, -60000.f), 60000.f)));
                // The reference point of the exponentials moves only when the row maximum has grown by more than 2^8
                // (P could leave the fp16 range); the final division by the row sum makes the result independent of it.
                const bool grow = bmax > m_run + kRescaleStep;   // also true for the first finite score of a row
                if (j > 0) {
                    // P_{j-1} V_{j-1} has completed: it was issued before this block's Q K^T by the same thread, and the
                    // commit that signalled S_j covers every earlier operation of that thread.
                    if (__any_sync(0xffffffffu, grow)) {
                        // O and the running sum move to the new reference point (0 when the row had nothing before)
                        const float alpha = grow ? ((m_run == -INFINITY) ? 0.f : ex2_fast(m_run - bmax)) : 1.f;
                        l_run *= alpha;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t o[16];
                            tmem_ld16(o_addr + c * 16, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st16(o_addr + c * 16, o);
                        }
                    }
                }
                if (grow) m_run = bmax;
                if (tid == 0) AT_STAMP(31 + 4 * (j & 3));
                // P = 2^(s - reference) as packed fp16 over the first 32 score columns; the row sum is the sum of exactly
                // the fp16 values that are multiplied with V.
                const float nshift = (m_run == -INFINITY) ? 0.f : -m_run;
#pragma unroll
                for (int c = 0; c < kNCh; ++c) {
                    uint32_t pk[16];
                    if (plain && kScoresF16) {
                        const half2 sc2 = __float2half2_rn(p.scale_log2), sh2 = __float2half2_rn(nshift);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const half2 a2 = __hfma2(*reinterpret_cast<const half2*>(&rp[c * 16 + i]), sc2, sh2);
                            pk[i] = ex2_h2(*reinterpret_cast<const uint32_t*>(&a2));
                        }
                    } else if (plain) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            pk[i >> 1] = ex2_h2(pack2(fmaf(__uint_as_float(rf[c][i]), p.scale_log2, nshift),
                                                      fmaf(__uint_as_float(rf[c][i + 1]), p.scale_log2, nshift)));
                    } else {
                        float v[32];
                        general_chunk(c, v);
#pragma unroll
                        for (int i = 0; i < 32; i += 2) pk[i >> 1] = ex2_h2(pack2(v[i] + nshift, v[i + 1] + nshift));
                    }
                    tmem_st16(p_addr + c * 16, pk);
                    l_run += sum_packed(pk);
                }
                if (tid == 0) AT_STAMP(32 + 4 * (j & 3));
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (elect_one()) mbar_arrive(&sh->p_ready);
                if (tid == 0) AT_STAMP(33 + 4 * (j & 3));
            }
            // ---- epilogue: O / row sum -> fp16 -> global
            const bool fin = ok && !sh->abort && mbar_wait(&sh->o_done, 0);
            tc_fence_after();
            if (tid == 0) AT_STAMP(50);
            if (fin) {
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                half* zrow = p.Z + (size_t)(tok0 + qr) * p.z_pitch + h * kHD;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[16];
                    tmem_ld16(o_addr + c * 16, r);
                    tmem_ld_wait();
                    if (qr < L) {
                        uint4 o[2];
                        uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            ow[i] = pack2(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
                        *reinterpret_cast<uint4*>(zrow + c * 16) = o[0];
                        *reinterpret_cast<uint4*>(zrow + c * 16 + 8) = o[1];
                    }
                }
            } else if (lane == 0 && !sh->abort) {
                atomicExch(p.err, 22);
                sh->abort = 1;
            }
        }
    } else if (b >= 0 && warp < 4) {
        // no valid key: the output rows are zero
        const int qr = q0 + warp * 32 + lane;
        if (qr < L) {
            uint4* z = reinterpret_cast<uint4*>(p.Z + (size_t)(tok0 + qr) * p.z_pitch + h * kHD);
#pragma unroll
            for (int i = 0; i < 8; ++i) z[i] = make_uint4(0, 0, 0, 0);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) AT_STAMP(51);
    if (warp == kSoftmaxWarps) tmem_dealloc(tmem, kTmemCols);
}

long long* g_attn_prof = nullptr;
bool g_scores_fp32 = false;   // how Q K^T is accumulated (see kScoresF16 above); process-wide, read at launch

// Error word of the kernel's bounded waits: a device variable of the library image (one copy per device that
// loads the library, zero at load), so that no launch ever allocates. The kernel writes it only when a wait
// gives up. In host code the symbol is a handle, not an address: the address is looked up once per device.
__device__ int g_attn_err_word;
constexpr int kMaxDevices = 64;
std::mutex g_err_mu;
int* g_err_ptr[kMaxDevices] = {nullptr};

int attn_err_address(int** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e, "attention: cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(ET_ERR_UNSUPPORTED, "attention: device ordinal above 63");
    std::lock_guard<std::mutex> lk(g_err_mu);
    if (!g_err_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attn_err_word);
        if (e != cudaSuccess) return cuda_status(e, "attention: cudaGetSymbolAddress");
        g_err_ptr[dev] = static_cast<int*>(p);
    }
    *out = g_err_ptr[dev];
    return ET_OK;
}

}  // namespace

// Looks up the error word's address on the current device (encoder constructors call this so that the first
// launch, possibly inside a caller's stream capture, has nothing left to set up).
int attention_prepare_device() {
    int* p = nullptr;
    return attn_err_address(&p);
}

// Fast path. Returns ET_ERR_UNSUPPORTED (without touching anything) when the case is outside its range, so the
// caller can use the general kernel instead.
int attention_tc_launch(half* Z, const half* Q, const half* K, const half* V, int q_pitch, int v_pitch,
                        const half* mask, int mask_ld, const int* cu_seqlens, const int* valid_lens, int batch,
                        int uniform_len, int total_tokens, int max_len, int d_model, int nhead, cudaStream_t st) {
    if (d_model / nhead != kHD || d_model % nhead) return ET_ERR_UNSUPPORTED;
    if (max_len <= 0) return ET_ERR_UNSUPPORTED;   // longest sequence unknown: the caller uses the general kernel
    if ((q_pitch & 7) || (v_pitch & 7) || (d_model & 7) || !aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(Z))
        return ET_ERR_UNSUPPORTED;
    if (batch <= 0 || total_tokens <= 0) return ET_OK;
    int* err_word = nullptr;
    {
        const int rc = attn_err_address(&err_word);
        if (rc) return rc;
    }
    CUtensorMap tq, tk, tv;
    const uint64_t rows = (uint64_t)total_tokens;
    // the column extent covers all heads of the operand; Q/K/V may be slices of one fused [tokens x 3 d_model] buffer
    if (!make_tmap_2d_f16(&tq, Q, rows, (uint64_t)d_model, (uint64_t)q_pitch, kBQ, kHD, 128) ||
        !make_tmap_2d_f16(&tk, K, rows, (uint64_t)d_model, (uint64_t)q_pitch, kBK, kHD, 128) ||
        !make_tmap_2d_f16(&tv, V, rows, (uint64_t)d_model, (uint64_t)v_pitch, kBK, kHD, 128))
        return fail(ET_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed");
    TcParams p;
    p.Z = Z; p.mask = mask; p.cu_seqlens = cu_seqlens; p.valid_lens = valid_lens;
    p.z_pitch = d_model; p.mask_ld = mask_ld; p.batch = batch; p.uniform_len = uniform_len;
    p.scale_log2 = kLog2e / sqrtf((float)kHD);
    p.err = err_word;
    p.prof = g_attn_prof;
    const size_t smem = (size_t)kTile + 4 * (size_t)kKVTile + sizeof(TcShared) + 1024;
    static PerDeviceOnce once;
    const cudaError_t attr_err = once.run([] {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
        if (e != cudaSuccess) return e;
        return cudaFuncSetAttribute(attention_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    });
    if (attr_err != cudaSuccess) return cuda_status(attr_err, "attention: shared memory opt-in");
    const int nblk = cu_seqlens ? (total_tokens + kBQ - 1) / kBQ + batch : batch * ((uniform_len + kBQ - 1) / kBQ);
    auto kernel = g_scores_fp32 ? attention_tc_kernel<false> : attention_tc_kernel<true>;
    return cuda_status(launch_pdl(kernel, dim3(nblk, nhead), dim3(kThreads), smem, st, tq, tk, tv, p),
                       "attention (tcgen05) launch");
}

void attention_tc_set_profile_buffer(long long* dev_buf) { g_attn_prof = dev_buf; }

void attention_tc_set_scores_fp32(int on) { g_scores_fp32 = on != 0; }
int attention_tc_scores_fp32() { return g_scores_fp32 ? 1 : 0; }

// Reads and clears the current device's error word of the tcgen05 attention kernel (synchronises).
// 0 = no wait gave up since the last read.
int attention_tc_error(int* code) {
    *code = 0;
    int* word = nullptr;
    int rc = attn_err_address(&word);
    if (rc) return rc;
    cudaError_t e = cudaMemcpy(code, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_status(e, "attention error read");
    if (*code) {
        e = cudaMemset(word, 0, sizeof(int));
        if (e != cudaSuccess) return cuda_status(e, "attention error clear");
    }
    return ET_OK;
}

}  // namespace et
