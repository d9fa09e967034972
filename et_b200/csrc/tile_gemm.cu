// Tile-sparse linear  Y[T x N] = X[T x K] . W^T + bias  (optional tanh-GELU), W in 16x16 tile-BSR.
// Replaces kernels/linear.cu:54-167 of the reference (both kernels and both launchers) and the
// weight side of encoder/Linear.h:4-46.
//
// sm_100a design (tcgen05 + TMEM + TMA), zero tiles are never touched:
//   * A CTA owns a slab of 128 tokens and a chunk of up to 24 output block-rows (16 features each).
//     Its fp32 accumulators live in tensor memory: 16 TMEM columns per block-row, 384 columns at most.
//   * The activations are the A operand and are read from tensor memory, not shared memory: X is
//     brought in by TMA (two 128-byte-swizzled 128 x 64 panels per 128-wide K chunk) and moved
//     smem -> TMEM with tcgen05.cp into one of 2-4 64-column slots. With A in TMEM a 128x16x16 UMMA no
//     longer pays the 4 KB shared-memory read of A, which otherwise bounds small-N UMMAs to ~20 % of peak.
//   * Every kept tile is one UMMA  D[128 x 16] += A[128 x 16] . tile^T  (B operand = the tile in
//     shared memory, canonical no-swizzle K-major layout). A single warp can only issue one UMMA per
//     ~55 clocks, so eight warps issue concurrently, each owning a disjoint set of block-rows.
//   * The weight is re-packed once, on the host, into a stream of blocks, one per (block-row chunk,
//     128-wide K chunk): a per-warp issue list followed by the tiles already in UMMA layout. One
//     cp.async.bulk brings a block into shared memory. The sparsity pattern is kept exactly.
//   * Persistent CTAs (grid = min(tiles, SMs)); one chunk counter runs on across a CTA's tiles and indexes three
//     rings, one per resource, because the operands live for different times: shared-memory slots for activations
//     (free once copied on to tensor memory), shared-memory slots for weight blocks (free once their UMMAs have
//     completed), tensor-memory A slots (free once the UMMAs that read them have been issued: tcgen05 operations
//     execute in issue order). Roles: warp 0 copies activations, warp 1 weight blocks, warps 2-3 move activations
//     to tensor memory, warps 4-11 issue UMMAs. (Every asynchronous operation costs the issuing warp 100-250
//     clocks, so the hops per chunk are what the loop time is made of.)
//   * Epilogue, warp by warp, by sixteen warps (the eight issuers and eight helpers that sleep on a hardware
//     barrier during the main loop): tcgen05.ld, + bias, optional GELU, fp16, staged in the warp's own
//     64-byte-swizzled 32 x 32 buffer and written with one TMA store (rows beyond T and columns beyond N are clipped).
//   * Every wait is executed by all lanes of the waiting warp (no polling lane and shuffle), and no role reads the
//     CTA's abort flag inside its loop: both were measured to cost ~10 % and ~3 % of the kernel's time.
// Every mbarrier wait is bounded; a wait that gives up records a code in the error word, the CTA
// stops issuing, frees its tensor memory and returns.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>
#include "common.h"
#include "ptx.cuh"
#include "tmap.h"
#include "tile_gemm.h"

namespace et {

namespace {

constexpr int kSlab = 128;          // tokens per CTA
constexpr int kKC = 128;            // K elements per chunk = two 128-byte-swizzled 64-column panels
constexpr int kPanel = 64;          // columns per panel
constexpr int kSlices = kKC / 16;   // UMMA K steps per chunk
constexpr int kMaxNB = 24;          // block-rows per CTA (384 accumulator columns)
constexpr int kSlotCols = kKC / 2;  // TMEM columns of one A slot
constexpr int kMaxRing = 6;           // barriers per ring
constexpr int kIssuers = 8;         // UMMA-issuing warps; they also take a share of every epilogue
constexpr int kHelpers = 8;         // warps that only work in the epilogue (asleep on a hardware barrier otherwise)
constexpr int kProducers = 2;       // warp 0 copies activations, warp 1 weight blocks
constexpr int kMovers = 2;          // tcgen05.cp-issuing warps, taking chunks in turn
constexpr int kFirstMover = kProducers;
constexpr int kFirstIssuer = kFirstMover + kMovers;
constexpr int kFirstHelper = kFirstIssuer + kIssuers;
constexpr int kEpiWarps = kIssuers + kHelpers;
constexpr int kEpiPerQuarter = kEpiWarps / 4;   // warps that share the 32 rows of a tensor-memory lane quarter
constexpr int kThreads = 32 * (kFirstHelper + kHelpers);
constexpr int kDirInParams = 32;    // directory entries of each chunk's first block travel as kernel parameters
constexpr int kUnitCols = 32;          // columns per epilogue store
constexpr int kUnitBytes = 32 * kUnitCols * 2;   // one warp's staging buffer: 32 rows x 32 columns
constexpr int kPanelBytes = kSlab * kPanel * 2;   // 16 KB
constexpr int kXStageBytes = kSlab * kKC * 2;     // 32 KB
constexpr int kHeaderBytes = 64;
constexpr int kSmemMax = 232448;    // 227 KB: the per-CTA opt-in limit of sm_100
constexpr int kMaxKChunks = 256;    // in_feat up to 32768

struct GemmParams {
    const uint2* dir;        // per (chunk, k-chunk): {offset, size} in 16-byte units
    const uint8_t* stream;   // packed blocks
    half* Y;
    const half* bias;
    int T, N, k_chunks, n_chunks, n_tiles, nb, stage_b_bytes, nx, nw, a_slots, gelu;
    int* err;
    uint2 first[kDirInParams];   // dir[chunk][0] for chunk < kDirInParams: no global load before the first TMA
    GemmFusion fz;           // LayerNorm folded into the epilogue (modes 1-3 of the kernel template)
    long long* prof;         // optional per-role clock64 stamps of CTA (0,0) (ET_GEMM_PROFILE builds only)
};

#ifdef ET_GEMM_PROFILE
#define ET_STAMP(slot) do { if (p.prof && blockIdx.x == 0 && blockIdx.y == 0) p.prof[(slot)] = clock64(); } while (0)
#else
#define ET_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ void tc_cp_128x256b(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.128x256b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tmem_st16_zero(uint32_t taddr) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr),
        "r"(0u)
        : "memory");
}
// tanh-GELU of two values in packed fp16 arithmetic: 0.5 x (1 + tanh(x (c1 + c2 x^2))), six packed operations and
// one special-function op per pair, no conversion. The epilogue is bound by the conversion unit (fp32 <-> fp16
// conversions and special functions run at 16 per clock per SM): with the polynomial in fp32 and conversions
// around the tanh a 128 x 384 GELU tile took ~9000 clocks against ~4400 without GELU. The result is stored as fp16
// anyway; tanh saturates, so the rounding of its argument does not grow with |x| (an argument that overflows to
// infinity gives tanh = +-1, the correct limit).
__device__ __forceinline__ half2 gelu_tanh_h2(half2 x) {
    const half2 c1 = __float2half2_rn(0.7978845608028654f), c2 = __float2half2_rn(0.7978845608028654f * 0.044715f);
    const half2 u = __hmul2(x, __hfma2(__hmul2(x, x), c2, c1));
    uint32_t t;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(*reinterpret_cast<const uint32_t*>(&u)));
    const half2 hx = __hmul2(x, __float2half2_rn(0.5f));
    return __hfma2(hx, *reinterpret_cast<const half2*>(&t), hx);
}

struct Shared {
    // Barrier rings (a parity wait is only safe for a waiter that has seen the barrier's previous phase complete and
    // cannot be a whole phase late, which fixes each ring's length):
    uint64_t full_x[kMaxRing];    // [chunk % FX]  the chunk's activations have landed (TMA); FX = nx, doubled when odd, so
                                  //               that a barrier always falls to the same one of the two movers
    uint64_t full_w[kMaxRing];    // [chunk % FW]  the chunk's weight block has landed (bulk copy); FW from nw likewise
    uint64_t a_ready[kMaxRing];   // [chunk % kMaxRing]  the chunk's activations are in tensor memory (mover commit): read by
                                  //               the issuers, and by the activation producer as "shared-memory slot free"
    uint64_t a_issued[kMaxRing];  // [chunk % a_slots]  every issuer has issued (not completed) its UMMAs on the chunk
    uint64_t done[kMaxRing];      // [chunk % nw]  every issuer's UMMAs on the chunk have completed (8 commits)
    uint64_t acc_done;            // 8 issuer commits after a tile's last chunk
    uint32_t tmem_base;
    volatile int abort;            // any role gave up: everybody winds down
    volatile int issuer_abort[2];  // [tile parity]: set by an issuer warp that gives up during a tile, read by
                                   // all of them after the named barrier that opens the next tile, so that
                                   // the eight warps leave the tile loop at the same tile
    __align__(16) half bias[2][kMaxNB * 16];  // [tile parity]: a warp may still convert tile t while another
                                              // stages the bias of tile t + 1
};

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// One 32-column unit of the epilogue, in three steps so that two units can be in flight per warp.
__device__ __forceinline__ void epi_load(uint32_t taddr, bool two, uint32_t (&acc)[32]) {
    if (two) {
        tmem_ld32(taddr, acc);
    } else {
        uint32_t lo[16];
        tmem_ld16(taddr, lo);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            acc[i] = lo[i];
            acc[16 + i] = 0u;
        }
    }
}
template <bool kGelu>
__device__ __forceinline__ void epi_convert(const uint32_t (&acc)[32], const half* bias, bool two, uint4 (&ov)[4]) {
    uint4 bv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
        bv[c] = (two || c < 2) ? reinterpret_cast<const uint4*>(bias)[c] : make_uint4(0u, 0u, 0u, 0u);
    const half2* bh = reinterpret_cast<const half2*>(bv);
    half2* oh = reinterpret_cast<half2*>(ov);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        if constexpr (kGelu) {
            // one conversion per pair: the accumulator is packed first and the bias is added in packed fp16
            oh[i] = gelu_tanh_h2(__hadd2(__floats2half2_rn(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1])), bh[i]));
        } else {
            const float2 bb = __half22float2(bh[i]);
            oh[i] = __floats2half2_rn(__uint_as_float(acc[2 * i]) + bb.x, __uint_as_float(acc[2 * i + 1]) + bb.y);
        }
    }
}
// Row `lane` of a 32 x 32 unit: four 16-byte chunks under the 64-byte swizzle (chunk ^= (row / 2) % 4).
__device__ __forceinline__ void epi_write(uint8_t* buf, int lane, const uint4 (&ov)[4]) {
    uint8_t* prow = buf + lane * 64;
    const int x = (lane >> 1) & 3;
#pragma unroll
    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(prow + ((c ^ x) << 4)) = ov[c];
}

// ---- LayerNorm folded into the epilogue (the layer stack's fused path) --------------------------------------------
// A residual-add + LayerNorm between two linears costs two passes over the activations. Folded: the linear BEFORE
// the LayerNorm adds the residual in its epilogue, writes the un-normalised sum y and, per row and CTA, the partial
// sums (sum y, sum y^2) of its columns (modes 2 and 3); the linear AFTER it reads y with gamma multiplied into its
// weights and applies mean and 1/std per row in its epilogue (mode 1):
//     LN(y) W^T + b = r (y (gamma o W)^T - mu c) + d,   c_n = sum_k gamma_k W_nk,  d_n = sum_k beta_k W_nk + b_n.
// Partial sums are written to their own slot per (row, column chunk, warp of the row quarter) and added up by the
// reader in slot order: no atomics, results do not depend on scheduling.
__device__ __forceinline__ void row_stats(const float* __restrict__ st, int np, int row, float inv_d, float eps,
                                          float& r, float& rmu) {
    float s1 = 0.f, s2 = 0.f;
    const float2* ps = reinterpret_cast<const float2*>(st) + (size_t)row * np;
    for (int i = 0; i < np; ++i) {
        const float2 v = __ldg(ps + i);
        s1 += v.x;
        s2 += v.y;
    }
    const float mu = s1 * inv_d;
    r = rsqrtf(fmaxf(s2 * inv_d - mu * mu, 0.f) + eps);
    rmu = r * mu;
}
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// One 32-column unit in a fused mode. Mode 1: (ra, rb) = (1/std, mean/std) of this thread's row of the input.
// Modes 2, 3: y = acc + bias + residual, (s1, s2) += (y, y^2); in mode 3 the residual is the LayerNorm of the row of
// `resid` with (ra, rb) = (1/std, mean/std) of that row and gamma_s / beta_s.
// This thread's 32 residual values of a unit (64 bytes of its row) as two 32-byte loads; zeros outside the tensor.
__device__ __forceinline__ void resid_load(uint32_t (&r)[16], const half* __restrict__ resid, int N, int col0, int row, bool row_ok) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        if (row_ok && col0 + 16 * hh < N) {
            const half* src = resid + (size_t)row * N + col0 + 16 * hh;
            asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(r[8 * hh]), "=r"(r[8 * hh + 1]), "=r"(r[8 * hh + 2]), "=r"(r[8 * hh + 3]), "=r"(r[8 * hh + 4]),
                           "=r"(r[8 * hh + 5]), "=r"(r[8 * hh + 6]), "=r"(r[8 * hh + 7])
                         : "l"(src));
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[8 * hh + i] = 0u;
        }
    }
}

template <bool kGelu, int kMode>
__device__ __forceinline__ void epi_fused(const uint32_t (&acc)[32], const uint32_t (&rsd)[16], const GemmFusion& f, int N, int col0,
                                          float ra, float rb, float& s1, float& s2, uint4 (&ov)[4]) {
    half2* oh = reinterpret_cast<half2*>(ov);
#pragma unroll
    for (int c = 0; c < 4; ++c) {      // eight columns at a time
        const int col = col0 + 8 * c;
        float v[8];
        if (col < N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[8 * c + i]);
            if constexpr (kMode == 1) {
                const float4 c0 = ldg4(f.colc + col), c1 = ldg4(f.colc + col + 4), d0 = ldg4(f.cold + col), d1 = ldg4(f.cold + col + 4);
                const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float dd[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = fmaf(ra, v[i], fmaf(-rb, cc[i], dd[i]));
            } else {
                const float4 b0 = ldg4(f.bias_f32 + col), b1 = ldg4(f.bias_f32 + col + 4);
                const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                const half2* h2 = reinterpret_cast<const half2*>(&rsd[4 * c]);
                float res[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 t = __half22float2(h2[i]);
                    res[2 * i] = t.x;
                    res[2 * i + 1] = t.y;
                }
                if constexpr (kMode == 3) {
                    const float4 g0 = ldg4(f.gamma_s + col), g1 = ldg4(f.gamma_s + col + 4), e0 = ldg4(f.beta_s + col), e1 = ldg4(f.beta_s + col + 4);
                    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                    const float ee[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) res[i] = fmaf(fmaf(res[i], ra, -rb), gg[i], ee[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i] += bb[i] + res[i];
                    s1 += v[i];
                    s2 = fmaf(v[i], v[i], s2);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const half2 hp = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            oh[4 * c + i] = kGelu ? gelu_tanh_h2(hp) : hp;
        }
    }
}

// Persistent: CTA c processes tiles c, c + gridDim.x, ... (tile = slab * n_chunks + chunk, so CTAs that run
// together share activations in L2). One chunk counter runs on across tiles and indexes three rings:
//   * nx shared-memory slots of 32 KB for the activations of a chunk, free as soon as the movers' tcgen05.cp of the
//     chunk have completed (the movers' one commit per chunk, `a_ready`, is read by the issuers and by the
//     activation producer);
//   * nw shared-memory slots for the weight block of a chunk, free when the chunk's UMMAs have completed (`done`);
//   * a_slots tensor-memory slots for the A operand, free when the UMMAs of the chunk a_slots earlier have been
//     issued (`a_issued`).
// What bounds the chunk period is bytes in flight per clock of lifetime; each operand gets the slots its own
// lifetime needs. Every role does as few serial barrier operations per chunk as possible: on this part a wait on a
// completed mbarrier, a tcgen05.cp or a TMA issue each cost a warp 100-250 clocks.
// While the sixteen epilogue warps convert and store one tile, the producers and the movers stage the next tile's
// first chunks.
template <bool kGelu, int kMode>
__global__ void __launch_bounds__(kThreads, 1)
tile_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int NX = p.nx, NW = p.nw, RA = p.a_slots;
    const int FX = (NX & 1) ? 2 * NX : NX, FW = (NW & 1) ? 2 * NW : NW;
    uint8_t* const xring = smem;                                       // NX x 32 KB of activations
    uint8_t* const wring = smem + (size_t)NX * kXStageBytes;           // NW weight blocks
    uint8_t* const epi = wring + (size_t)NW * p.stage_b_bytes;         // 16 warps x 2 KB
    Shared* sh = reinterpret_cast<Shared*>(epi + kEpiWarps * kUnitBytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x;
    const uint32_t a_col0 = 512u - (uint32_t)(RA * kSlotCols);
    const int my_tiles = (p.n_tiles - (int)blockIdx.x + G - 1) / G;
    if (tid == 0) ET_STAMP(0);
    // The next kernel in the stream is released late, when this CTA's last main loop is over: a dependent CTA
    // that becomes resident earlier would hold an SM while it waits for this whole grid, an SM that a kernel of
    // another stream (another batch in flight) could use.

    if (warp == 0) {
        // ---------------- activation producer: lane 0 issues the copies, lane 1 polls (a wait by the thread that has
        // just issued a bulk copy costs several hundred clocks)
        if (lane < kMaxRing) mbar_init(&sh->full_x[lane], 1);
        else if (lane < 2 * kMaxRing) mbar_init(&sh->full_w[lane - kMaxRing], 1);
        else if (lane < 3 * kMaxRing) mbar_init(&sh->a_ready[lane - 2 * kMaxRing], 1);
        else if (lane < 4 * kMaxRing) mbar_init(&sh->a_issued[lane - 3 * kMaxRing], kIssuers);
        else if (lane < 5 * kMaxRing) mbar_init(&sh->done[lane - 4 * kMaxRing], kIssuers);
        else if (lane == 5 * kMaxRing) mbar_init(&sh->acc_done, kIssuers);
        static_assert(5 * kMaxRing < 32, "one lane per barrier");
        if (lane <= 5 * kMaxRing) fence_mbar_init();
        if (lane == 0) {
            sh->abort = 0;
            sh->issuer_abort[0] = 0;
            sh->issuer_abort[1] = 0;
        }
        __syncwarp();
        named_barrier_arrive(4, 64);         // the weight producer may start
        named_barrier_arrive(2, kThreads);   // barriers are initialised: release the other warps
        if (lane == 0) ET_STAMP(8);
        // Everything above touched only this kernel's own resources. The activations may still be in the making:
        // wait for the preceding kernels before the first copy (lane 0 issues them all).
        if (lane == 0) pdl_wait();
        int issued = 0, xs = 0, fx = 0, ar = 0;
        uint32_t pha = 0;
        bool alive = true;
        for (int tl = 0; tl < my_tiles && alive; ++tl) {
            const int tile = (int)blockIdx.x + tl * G;
            const int slab = tile / p.n_chunks;
            for (int kc = 0; kc < p.k_chunks; ++kc) {
                // the slot is free when the chunk NX before this one has been copied on to tensor memory
                const bool go = issued < NX || mbar_wait(&sh->a_ready[ar], pha);
                if (lane == 0 && issued < 64) ET_STAMP(900 + issued);
                if (!go) {
                    if (lane == 0 && !sh->abort) {
                        atomicExch(p.err, 11);
                        sh->abort = 1;
                    }
                    alive = false;
                    break;
                }
                if (lane == 0) {
                    mbar_expect_tx(&sh->full_x[fx], kXStageBytes);
                    tma_load_3d(xring + (size_t)xs * kXStageBytes, &tmX, 0, slab * kSlab, kc * (kKC / kPanel),
                                &sh->full_x[fx]);   // both panels, one op
                    if (issued < 64) ET_STAMP(100 + issued);
                }
                if (issued >= NX && ++ar == kMaxRing) { ar = 0; pha ^= 1u; }
                ++issued;
                if (++fx == FX) fx = 0;
                if (++xs == NX) xs = 0;
            }
        }
        // Leaving early: wait (bounded) for the copies still in flight before the CTA exits.
        if (lane == 1 && sh->abort)
            for (int kk = issued > NX ? issued - NX : 0; kk < issued; ++kk)
                mbar_wait(&sh->full_x[kk % FX], (uint32_t)(kk / FX) & 1u);
    } else if (warp == 1) {
        // ---------------- weight producer: the packed weight does not depend on the preceding kernel, so these copies
        // start as soon as the barriers exist. A slot is free when the UMMAs that read it have completed.
        named_barrier_sync(4, 64);
        named_barrier_arrive(2, kThreads);
        int issued = 0, ws = 0, fw = 0;
        uint32_t phw = 0;
        bool alive = true;
        for (int tl = 0; tl < my_tiles && alive; ++tl) {
            const int tile = (int)blockIdx.x + tl * G;
            const int chunk = tile % p.n_chunks;
            const uint2* gdir = p.dir + (size_t)chunk * p.k_chunks;
            // directory entries: the first one of the first tile comes from the kernel parameters, the others are
            // fetched one chunk ahead
            uint2 dnext = (tl == 0 && chunk < kDirInParams) ? p.first[chunk] : (lane == 0 ? __ldg(gdir) : make_uint2(0, 0));
            for (int kc = 0; kc < p.k_chunks; ++kc) {
                const uint2 d = dnext;
                if (lane == 0 && kc + 1 < p.k_chunks) dnext = __ldg(gdir + kc + 1);
                const bool go = mbar_wait(&sh->done[ws], phw ^ 1u);
                if (!go) {
                    if (lane == 0 && !sh->abort) {
                        atomicExch(p.err, 15);
                        sh->abort = 1;
                    }
                    alive = false;
                    break;
                }
                if (lane == 0) {
                    const uint32_t bbytes = d.y * 16u;
                    mbar_expect_tx(&sh->full_w[fw], bbytes);
                    bulk_load(wring + (size_t)ws * p.stage_b_bytes, p.stream + (size_t)d.x * 16u, bbytes, &sh->full_w[fw]);
                    if (issued < 64) ET_STAMP(1100 + issued);
                }
                ++issued;
                if (++fw == FW) fw = 0;
                if (++ws == NW) { ws = 0; phw ^= 1u; }
            }
        }
        if (lane == 1 && sh->abort)
            for (int kk = issued > NW ? issued - NW : 0; kk < issued; ++kk)
                mbar_wait(&sh->full_w[kk % FW], (uint32_t)(kk / FW) & 1u);
    } else {
        if (warp == kFirstMover) {
            tmem_alloc(&sh->tmem_base, 512);
            tmem_relinquish();
        }
        tc_fence_before();
        named_barrier_sync(1, kThreads - 32 * kProducers);   // all but the producers: the tensor-memory base is visible
        tc_fence_after();
        const uint32_t tmem = sh->tmem_base;
        // Accumulators start at zero: block-rows without tiles are legal and every UMMA accumulates. (After
        // each tile the epilogue clears what it has read.)
        if (warp >= kFirstIssuer) {
            const int w = warp - kFirstIssuer;
            const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
            for (int br = (w >> 2); br < p.nb; br += kEpiPerQuarter) tmem_st16_zero(tmem + lane_base + br * 16);
            tmem_st_wait();
        }
        tc_fence_before();
        named_barrier_sync(2, kThreads);        // + the producers' arrives: mbarriers are initialised
        tc_fence_after();
        if (tid == 32 * kFirstMover) ET_STAMP(2);
        const int n_items = my_tiles * p.k_chunks;

        if (warp < kFirstIssuer) {
            // ---------------- movers: shared memory -> tensor memory copy of the A operand. The mover warps take
            // chunks in turn; lane 1 polls, lane 0 issues and commits. The tensor-memory slot is free as soon as the
            // issuers have ISSUED the UMMAs of the chunk a_slots earlier: tcgen05 operations execute in issue order
            // (the order across threads being established by the fence + barrier pair), so the copy cannot overtake
            // the UMMAs that still read the slot, and the hop "UMMAs completed -> seen by the mover" (~500 clocks)
            // leaves the slot's cycle. The one commit per chunk tells the issuers that A is in place and the
            // activation producer that the shared-memory slot may be overwritten.
            const int m = warp - kFirstMover;
            int xs = m % NX, a = m % RA, fx = m, fw = m, ar = m;
            uint32_t phx = 0, phw = 0;
            for (int it = m; it < n_items; it += kMovers) {
                bool got = mbar_wait(&sh->full_x[fx], phx);
                if (got && it >= RA) got = mbar_wait(&sh->a_issued[a], (uint32_t)(it / RA - 1) & 1u);
                if (lane == 0 && it < 64) ET_STAMP(700 + it);
                if (!got) {
                    if (lane == 0) atomicExch(p.err, 12);
                    sh->abort = 1;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t xa = smem_u32(xring + (size_t)xs * kXStageBytes);
                    const uint32_t ta = tmem + a_col0 + a * kSlotCols;
#pragma unroll
                    for (int sl = 0; sl < kSlices; ++sl)
                        tc_cp_128x256b(ta + sl * 8,
                                       make_smem_desc(xa + (sl >> 2) * kPanelBytes + (sl & 3) * 32, 16, 1024, 2));
                }
                // The issuers take "A is in place" to mean "the chunk is in place": the commit waits for the weight block,
                // whose copy started later (its slot is free only when UMMAs have completed); the tcgen05.cp run meanwhile.
                got = mbar_wait(&sh->full_w[fw], phw);
                if (!got) {
                    if (lane == 0) atomicExch(p.err, 12);
                    sh->abort = 1;
                    break;
                }
                if (lane == 0) {
                    umma_commit(&sh->a_ready[ar]);
                    if (it < 64) ET_STAMP(300 + it);
                }
                __syncwarp();
                xs = (xs + kMovers) % NX;
                a = (a + kMovers) % RA;
                fx += kMovers;
                if (fx >= FX) { fx -= FX; phx ^= 1u; }
                fw += kMovers;
                if (fw >= FW) { fw -= FW; phw ^= 1u; }
                ar += kMovers;
                if (ar >= kMaxRing) ar -= kMaxRing;
            }
        } else {
            // ---------------- issuers (one UMMA per kept tile, A from tensor memory) and epilogue helpers. All sixteen
            // warps share every tile's epilogue: its time is a chain of per-unit latencies in each warp (tensor-memory
            // load, conversion, fence, TMA store issue: ~730 clocks per 32-column unit) while the tensor pipe idles,
            // so four warps per lane quarter halve it; the stores themselves drain in the background.
            const bool issuer = warp < kFirstHelper;
            const int w = warp - kFirstIssuer;   // 0-7 issuers, 8-15 helpers
            const int q = warp & 3;   // the TMEM lane quarter this warp may read: rows 32q .. 32q + 31 of the slab
            const int h = w >> 2;     // which of the four warps of this row quarter
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            // B tile descriptor: no swizzle, 128 B between core matrices along K, 256 B along N.
            const uint64_t b_desc0 = make_smem_desc(0, 128, 256, 0);
            // this warp's output staging: 32 rows x 32 columns (64-byte rows, 64-byte swizzle)
            uint8_t* const buf = epi + (size_t)w * kUnitBytes;
            bool ok = true;
            int ws = 0, a = 0, ar = 0;
            uint32_t pha = 0;
            for (int tl = 0; tl < my_tiles; ++tl) {
                const int tile = (int)blockIdx.x + tl * G;
                const int slab = tile / p.n_chunks, chunk = tile - slab * p.n_chunks;
                half* const tbias = sh->bias[tl & 1];
                {
                    const int col0 = chunk * p.nb * 16;
                    for (int i = tid - 32 * kFirstIssuer; i < p.nb * 16; i += 32 * kEpiWarps)
                        tbias[i] = (col0 + i < p.N) ? p.bias[col0 + i] : __float2half(0.f);
                }
                // One rendezvous per tile: the bias is staged, every warp has cleared its accumulator columns,
                // and a warp that gave up in the previous tile is seen by all.
                named_barrier_sync(3, 32 * kEpiWarps);
                if (tl > 0 && sh->issuer_abort[(tl - 1) & 1]) break;
                tc_fence_after();
                if (issuer) {
                    for (int kc = 0; kc < p.k_chunks && ok; ++kc) {
                        // a_ready implies that the weight block has landed too: the movers waited for both copies.
                        const bool got = mbar_wait(&sh->a_ready[ar], pha);
                        if (!got) {
                            if (lane == 0) atomicExch(p.err, 13);
                            sh->abort = 1;
                            sh->issuer_abort[tl & 1] = 1;
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint8_t* blk = wring + (size_t)ws * p.stage_b_bytes;
                        const uint32_t hw = reinterpret_cast<const uint32_t*>(blk)[w];
                        const int e0 = hw & 0xffff, ne = hw >> 16;
                        const uint32_t n_entries = reinterpret_cast<const uint32_t*>(blk)[8];
                        const uint4* ent = reinterpret_cast<const uint4*>(blk + kHeaderBytes) + e0;
                        const uint32_t tiles16 = (smem_u32(blk) + kHeaderBytes + n_entries * 16u) >> 4;
                        const uint32_t abuf = tmem + a_col0 + a * kSlotCols;
#pragma unroll 4
                        for (int i = 0; i < ne; ++i) {
                            const uint4 en = ent[i];
                            if (elect_one())
                                umma_f16_ts(tmem + en.z, abuf + en.y, b_desc0 | (uint64_t)((tiles16 + en.x) & 0x3fff), en.w, 1u);
                        }
                        if (elect_one()) {
                            // issued: the tensor-memory slot may be refilled behind these UMMAs; completed: the weight slot
                            tc_fence_before();
                            mbar_arrive(&sh->a_issued[a]);
                            umma_commit(&sh->done[ws]);
                        }
                        if (w == 0 && lane == 0 && tl * p.k_chunks + kc < 64) ET_STAMP(600 + tl * p.k_chunks + kc);
                        __syncwarp();
                        if (++ws == NW) ws = 0;
                        if (++a == RA) a = 0;
                        if (++ar == kMaxRing) { ar = 0; pha ^= 1u; }
                    }
                    if (elect_one()) umma_commit(&sh->acc_done);
                    __syncwarp();
                    named_barrier_arrive(5, 32 * kEpiWarps);   // wakes the helpers: the tile's last UMMAs are on their way
                } else {
                    // asleep on a hardware barrier while the issuers run the main loop (polling warps would take issue
                    // slots and shared-memory bandwidth from the warps on the critical path)
                    named_barrier_sync(5, 32 * kEpiWarps);
                    if (sh->abort) {
                        sh->issuer_abort[tl & 1] = 1;
                        ok = false;
                    }
                }

                // ---------------- epilogue, warp by warp with no rendezvous: the four warps of a row quarter take the
                // tile's 32-column units in turn: TMEM -> registers -> bias / GELU (or a fused LayerNorm mode) -> fp16
                // -> the warp's own swizzled buffer -> TMA store.
                if (ok) {
                    const bool fin = mbar_wait(&sh->acc_done, (uint32_t)tl & 1u);
                    if (!fin) {
                        if (lane == 0) atomicExch(p.err, 14);
                        sh->abort = 1;
                        sh->issuer_abort[tl & 1] = 1;
                        ok = false;
                    }
                }
                tc_fence_after();
                if (tl + 1 == my_tiles) pdl_launch_dependents();   // its set-up overlaps this last epilogue
                if (w == 0 && lane == 0 && tl < 16) ET_STAMP(1400 + tl * 16);
                const int units = (p.nb + 1) >> 1;
                const bool more = tl + 1 < my_tiles;
                const int col0 = chunk * p.nb * 16, row0 = slab * kSlab + q * 32;
                const int row = row0 + lane;
                const bool row_ok = row < p.T;
                float ra = 0.f, rb = 0.f, s1 = 0.f, s2 = 0.f;
                if constexpr (kMode != 0) {
                    // fused modes: this thread's row statistics once per tile
                    if (ok && row_ok) {
                        if constexpr (kMode == 1) row_stats(p.fz.stats_in, p.fz.np_in, row, p.fz.inv_d_in, p.fz.eps, ra, rb);
                        if constexpr (kMode == 3) row_stats(p.fz.stats_src, p.fz.np_src, row, p.fz.inv_d_src, p.fz.eps, ra, rb);
                    }
                }
                // the residual of a unit is requested one unit ahead (64 bytes per thread straight from global
                // memory: the row-per-thread pattern touches whole 32-byte sectors)
                uint32_t rnext[16];
                if constexpr (kMode >= 2) {
                    if (ok && h < units) resid_load(rnext, p.fz.resid, p.N, col0 + h * kUnitCols, row, row_ok);
                }
                for (int u = h; u < units && ok; u += kEpiPerQuarter) {
                    const bool two = u * 2 + 1 < p.nb;
                    uint32_t acc[32];
                    epi_load(tmem + lane_base + u * 32, two, acc);
                    uint32_t rcur[16];
                    if constexpr (kMode >= 2) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) rcur[i] = rnext[i];
                        if (u + kEpiPerQuarter < units)
                            resid_load(rnext, p.fz.resid, p.N, col0 + (u + kEpiPerQuarter) * kUnitCols, row, row_ok);
                    }
                    tmem_ld_wait();
                    if (more) {   // clear what was just read, for the next tile
                        tmem_st16_zero(tmem + lane_base + u * 32);
                        if (two) tmem_st16_zero(tmem + lane_base + u * 32 + 16);
                    }
                    uint4 ov[4];
                    if constexpr (kMode == 0) epi_convert<kGelu>(acc, tbias + u * 32, two, ov);
                    else epi_fused<kGelu, kMode>(acc, rcur, p.fz, p.N, col0 + u * kUnitCols, ra, rb, s1, s2, ov);
                    // the buffer's previous store must have finished reading it (lane 0 issued it)
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
                    epi_write(buf, lane, ov);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (col0 + u * kUnitCols < p.N) tma_store_2d(&tmY, buf, col0 + u * kUnitCols, row0);
                        tma_store_commit();
                        if (w == 0 && tl < 16 && (u >> 2) < 14) ET_STAMP(1400 + tl * 16 + 1 + (u >> 2));
                    }
                }
                if constexpr (kMode >= 2) {
                    // this warp's share of the row: its own slot, written whether or not the warp had a unit
                    if (ok && row_ok)
                        reinterpret_cast<float2*>(p.fz.stats_out)[(size_t)row * p.fz.np_out + chunk * kEpiPerQuarter + h] = make_float2(s1, s2);
                }
                if (more) {
                    tmem_st_wait();
                    tc_fence_before();
                }
                if (w == 0 && lane == 0 && tl < 16) ET_STAMP(1400 + tl * 16 + 15);
            }
            if (lane == 0) tma_store_wait_read();   // shared memory may go once the stores have read it
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) ET_STAMP(4);
    if (warp == kFirstMover) tmem_dealloc(sh->tmem_base, 512);
}

}  // namespace

// --------------------------------------------------------------------------------- host side

struct TileWeight {
    int K = 0, N = 0, nb = 0, n_chunks = 0, k_chunks = 0, stage_b_bytes = 0, nx = 0, nw = 0, a_slots = 0;
    int tiles_per_cta = 1;   // > 1 when packed for SM time: a CTA takes that many tiles even when SMs are free
    long ntile = 0;
    int size_hint = 0;
    // the caller's arrays, kept so that weights can be concatenated (Q|K|V in one launch) and re-packed
    std::vector<int> h_row_ptr, h_row_offset;
    std::vector<half> h_data, h_bias;
    std::vector<uint2> h_first;   // directory entry of each chunk's first block
    uint2* d_dir = nullptr;
    uint8_t* d_stream = nullptr;
    half* d_bias = nullptr;
    float* d_bias_f32 = nullptr;                 // the bias as fp32 (fused epilogues)
    float* d_colc = nullptr; float* d_cold = nullptr;   // c_n, d_n of a weight folded with a LayerNorm's gamma / beta
    int* d_err = nullptr;
    size_t stream_bytes = 0;
};

// Ring depths for a chunk shape. The operands live for different times, so each has its own ring: an activation
// slot (32 KB) goes round in ~2700 clocks (free when copied on to tensor memory -> seen by the producer -> TMA ->
// landed -> copied), a weight slot in ~2500 (free when its UMMAs have completed -> seen -> bulk copy -> landed ->
// the issuers reach it), a tensor-memory slot in ~1400 (UMMAs issued -> seen by the mover -> eight tcgen05.cp ->
// seen by the issuers). The period of a chunk is the largest cycle / depth; shared memory is shared out to make
// that smallest (at most four slots per ring: beyond that the cycles above no longer bound the period).
struct RingShape { int nx, nw, a_slots; double period; };
static RingShape ring_shape(int nb, int stage_b_bytes) {
    const int tmem_slots = std::min(4, (512 - nb * 16) / kSlotCols);
    const int avail = kSmemMax - 1024 - (int)sizeof(Shared) - kEpiWarps * kUnitBytes;
    static_assert(kMovers == 2 && 2 * 3 <= kMaxRing && 4 <= kMaxRing, "the full-barrier rings must fit");
    RingShape best{0, 0, tmem_slots, 1e30};
    for (int nx = 2; nx <= 4; ++nx)
        for (int nw = 2; nw <= 4; ++nw) {
            if (nx * kXStageBytes + nw * stage_b_bytes > avail || tmem_slots < 1) continue;
            const double period = std::max({2700.0 / nx, 2500.0 / nw, 1400.0 / tmem_slots});
            if (period < best.period * 0.999) best = RingShape{nx, nw, tmem_slots, period};
        }
    return best;
}
// Block-rows per CTA from a model of the persistent kernel: a chunk takes the ring period, or its UMMAs (~10
// clocks each with eight issuing warps), or its share of L2 bandwidth (~64 bytes per clock per SM), whichever
// is longest; a tile ends with an epilogue of ~350 clocks per 32 columns and warp.
// What the pack optimises: 0 = the duration of one launch on an otherwise idle GPU (tiles spread over as many SMs
// as possible), 1 = SM time per launch (fewer, larger tiles: the right choice when several independent batches
// are in flight on separate streams and keep all SMs busy anyway).
static int g_goal = 0;
constexpr int kThroughputTilesPerCta = 2;
void tile_gemm_set_goal(int goal) { g_goal = goal == 1 ? 1 : 0; }

static int choose_nb(int n_block_rows, int k_chunks, int size_hint, double density) {
    const int slabs = std::max(1, (size_hint + kSlab - 1) / kSlab);
    const int sms = std::max(1, sm_count());
    double best = 0;
    int best_nb = 0;
    for (int nb : {24, 20, 16, 12, 8, 4}) {
        // chunks other than a single one must cover whole 64-column output panels (nb % 4 == 0)
        const int nbe = n_block_rows <= nb ? std::max(n_block_rows, 1) : nb;
        if (nbe > kMaxNB) continue;
        const double tiles_per_chunk = nbe * kSlices * density;
        // the largest block of a Bernoulli pattern: mean + 3 standard deviations
        const double tiles_max = std::min((double)nbe * kSlices,
                                          tiles_per_chunk + 3.0 * std::sqrt(nbe * kSlices * density * (1.0 - density)));
        const int stage_b = (int)((kHeaderBytes + tiles_max * 528.0 + 1023) / 1024) * 1024;
        const RingShape rs = ring_shape(nbe, stage_b);
        if (rs.nx < 2 || rs.a_slots < 1) continue;
        const long tiles = (long)slabs * ((n_block_rows + nbe - 1) / nbe);
        const double per_cta = (double)((tiles + sms - 1) / sms);
        const double t_chunk = std::max({rs.period, 10.0 * tiles_per_chunk,
                                         (kXStageBytes + tiles_per_chunk * 528.0) / 64.0});
        const double t_tile = k_chunks * t_chunk + 350.0 * ((nbe + 3) / 4) + 800.0;
        const double cost = g_goal == 1 ? (double)tiles * t_tile : per_cta * t_tile + 3000.0;
        if (best_nb == 0 || cost < best * 0.999) { best = cost; best_nb = nbe; }
    }
    return best_nb > 0 ? best_nb : std::min(8, std::max(n_block_rows, 1));
}

int tile_weight_pack(TileWeight** out, int K, int N, int size_hint, long ntile, const half* data,
                     const int* row_ptr, const int* row_offset, const half* bias, int nb_override) {
    if (!out) return fail(ET_ERR_INVALID, "tile weight: null output");
    *out = nullptr;
    if (K <= 0 || N <= 0 || K % 16 || N % 16) return fail(ET_ERR_INVALID, "tile weight: in/out features must be positive multiples of 16");
    if (ntile < 0 || !row_ptr || (ntile > 0 && (!row_offset || !data))) return fail(ET_ERR_INVALID, "tile weight: null array");
    const int NBR = N / 16;
    if (row_ptr[0] != 0 || row_ptr[NBR] != ntile) return fail(ET_ERR_INVALID, "tile weight: row_ptr does not span ntile");
    for (int r = 0; r < NBR; ++r)
        if (row_ptr[r + 1] < row_ptr[r]) return fail(ET_ERR_INVALID, "tile weight: row_ptr not monotone");
    for (long i = 0; i < ntile; ++i)
        if (row_offset[i] < 0 || row_offset[i] % 16 || row_offset[i] + 16 > K) return fail(ET_ERR_INVALID, "tile weight: row_offset out of range or not a multiple of 16");

    auto* w = new TileWeight();
    w->K = K; w->N = N; w->ntile = ntile; w->size_hint = size_hint;
    w->tiles_per_cta = g_goal == 1 ? kThroughputTilesPerCta : 1;
    const double density = (double)ntile / std::max(1.0, (double)NBR * (K / 16));
    w->nb = choose_nb(NBR, (K + kKC - 1) / kKC, size_hint, density);
    if (nb_override > 0) {
        const int nbo = std::min(nb_override, kMaxNB);
        w->nb = NBR <= nbo ? NBR : std::max(4, nbo / 4 * 4);
    }
    w->h_row_ptr.assign(row_ptr, row_ptr + NBR + 1);
    w->h_row_offset.assign(row_offset, row_offset + ntile);
    w->h_data.assign(data, data + (size_t)ntile * 256);
    w->h_bias.assign((size_t)N, __float2half(0.f));
    if (bias) std::copy(bias, bias + N, w->h_bias.begin());
    w->n_chunks = (NBR + w->nb - 1) / w->nb;
    w->k_chunks = (K + kKC - 1) / kKC;
    if (w->k_chunks > kMaxKChunks) { delete w; return fail(ET_ERR_UNSUPPORTED, "tile weight: in_feat above 32768"); }

    // Bucket tiles by (chunk, k-chunk, issuing warp).
    struct Ent { int tile; int slice; int lb; };
    const size_t nblocks = (size_t)w->n_chunks * w->k_chunks;
    std::vector<std::vector<Ent>> buckets(nblocks * kIssuers);
    for (int r = 0; r < NBR; ++r) {
        const int c = r / w->nb, lb = r % w->nb;
        for (int i = row_ptr[r]; i < row_ptr[r + 1]; ++i) {
            const int kc = row_offset[i] / kKC, sl = (row_offset[i] % kKC) / 16;
            buckets[((size_t)c * w->k_chunks + kc) * kIssuers + (lb % kIssuers)].push_back({i, sl, lb});
        }
    }
    std::vector<uint2> dir(nblocks);
    std::vector<uint8_t> stream;
    size_t max_block = 0;
    const uint32_t idesc16 = make_idesc_f16(128, 16);
    for (size_t b = 0; b < nblocks; ++b) {
        uint32_t n_entries = 0;
        for (int wv = 0; wv < kIssuers; ++wv) n_entries += (uint32_t)buckets[b * kIssuers + wv].size();
        const size_t bytes = kHeaderBytes + (size_t)n_entries * 16 + (size_t)n_entries * 512;
        const size_t off = stream.size();
        stream.resize(off + bytes, 0);
        uint32_t* hdr = reinterpret_cast<uint32_t*>(stream.data() + off);
        uint4* ent = reinterpret_cast<uint4*>(stream.data() + off + kHeaderBytes);
        uint8_t* tiles = stream.data() + off + kHeaderBytes + (size_t)n_entries * 16;
        uint32_t e = 0;
        for (int wv = 0; wv < kIssuers; ++wv) {
            auto& v = buckets[b * kIssuers + wv];
            std::stable_sort(v.begin(), v.end(), [](const Ent& a, const Ent& c) { return a.slice < c.slice; });
            if (e > 0xffff || v.size() > 0xffff) { delete w; return fail(ET_ERR_UNSUPPORTED, "tile weight: block too large"); }
            hdr[wv] = e | ((uint32_t)v.size() << 16);
            for (const Ent& t : v) {
                ent[e] = make_uint4(e * 32u, (uint32_t)t.slice * 8u, (uint32_t)t.lb * 16u, idesc16);
                const half* src = data + (size_t)t.tile * 256;
                uint8_t* dst = tiles + (size_t)e * 512;
                for (int n = 0; n < 16; ++n)
                    for (int k = 0; k < 16; ++k)
                        std::memcpy(dst + (n / 8) * 256 + (k / 8) * 128 + (n % 8) * 16 + (k % 8) * 2,
                                    src + n * 16 + k, 2);
                ++e;
            }
        }
        hdr[8] = n_entries;
        dir[b] = make_uint2((uint32_t)(off / 16), (uint32_t)(bytes / 16));
        max_block = std::max(max_block, bytes);
    }
    for (int c = 0; c < w->n_chunks && c < kDirInParams; ++c) w->h_first.push_back(dir[(size_t)c * w->k_chunks]);
    w->stage_b_bytes = (int)((max_block + 1023) / 1024 * 1024);
    {
        const RingShape rs = ring_shape(w->nb, w->stage_b_bytes);
        w->nx = rs.nx; w->nw = rs.nw; w->a_slots = rs.a_slots;
    }
    if (w->nx < 2 || w->a_slots < 1) { delete w; return fail(ET_ERR_UNSUPPORTED, "tile weight: weight block exceeds shared memory"); }
    w->stream_bytes = stream.size();

    cudaError_t e1 = cudaMalloc(&w->d_dir, dir.size() * sizeof(uint2));
    cudaError_t e2 = cudaMalloc(&w->d_stream, std::max<size_t>(stream.size(), 16));
    cudaError_t e3 = cudaMalloc(&w->d_bias, (size_t)N * sizeof(half));
    cudaError_t e4 = cudaMalloc(&w->d_err, sizeof(int));
    cudaError_t e5 = cudaMalloc(&w->d_bias_f32, (size_t)N * sizeof(float));
    if (e1 || e2 || e3 || e4 || e5) { tile_weight_free(w); return fail(ET_ERR_CUDA, "tile weight: cudaMalloc failed"); }
    {
        std::vector<float> bf((size_t)N, 0.f);
        if (bias) for (int i = 0; i < N; ++i) bf[i] = __half2float(bias[i]);
        cudaMemcpy(w->d_bias_f32, bf.data(), (size_t)N * sizeof(float), cudaMemcpyHostToDevice);
    }
    cudaMemcpy(w->d_dir, dir.data(), dir.size() * sizeof(uint2), cudaMemcpyHostToDevice);
    cudaMemcpy(w->d_stream, stream.data(), stream.size(), cudaMemcpyHostToDevice);
    if (bias) cudaMemcpy(w->d_bias, bias, (size_t)N * sizeof(half), cudaMemcpyHostToDevice);
    else cudaMemset(w->d_bias, 0, (size_t)N * sizeof(half));
    cudaMemset(w->d_err, 0, sizeof(int));
    int rc = cuda_status(cudaDeviceSynchronize(), "tile weight upload");
    if (rc) { tile_weight_free(w); return rc; }
    *out = w;
    return ET_OK;
}

// One weight whose output features are those of `parts` back to back (same in_feat): Q|K|V in one launch.
int tile_weight_concat(TileWeight** out, const TileWeight* const* parts, int count, int size_hint) {
    if (!out || !parts || count <= 0) return fail(ET_ERR_INVALID, "tile weight concat: bad arguments");
    std::vector<int> rp(1, 0), ro;
    std::vector<half> data, bias;
    int N = 0;
    for (int i = 0; i < count; ++i) {
        const TileWeight* w = parts[i];
        if (!w || w->K != parts[0]->K) return fail(ET_ERR_INVALID, "tile weight concat: in_feat differs");
        const int base = rp.back();
        for (size_t r = 1; r < w->h_row_ptr.size(); ++r) rp.push_back(base + w->h_row_ptr[r]);
        ro.insert(ro.end(), w->h_row_offset.begin(), w->h_row_offset.end());
        data.insert(data.end(), w->h_data.begin(), w->h_data.end());
        bias.insert(bias.end(), w->h_bias.begin(), w->h_bias.end());
        N += w->N;
    }
    return tile_weight_pack(out, parts[0]->K, N, size_hint > 0 ? size_hint : parts[0]->size_hint, (long)ro.size(), data.data(), rp.data(), ro.data(),
                            bias.data(), 0);
}

void tile_weight_free(TileWeight* w) {
    if (!w) return;
    cudaFree(w->d_dir); cudaFree(w->d_stream); cudaFree(w->d_bias); cudaFree(w->d_err);
    cudaFree(w->d_bias_f32); cudaFree(w->d_colc); cudaFree(w->d_cold);
    delete w;
}

static long long* g_prof = nullptr;
void tile_gemm_set_profile_buffer(long long* dev_buf) { g_prof = dev_buf; }

int tile_linear_run(const TileWeight* w, half* Y, const half* X, int T, int gelu, cudaStream_t st, const half* bias_dev,
                    const GemmFusion* fusion) {
    if (!w || !Y || !X) return fail(ET_ERR_INVALID, "tile linear: null pointer");
    if (T < 0) return fail(ET_ERR_INVALID, "tile linear: negative token count");
    if (T == 0) return ET_OK;
    if (!aligned16(X) || !aligned16(Y)) return fail(ET_ERR_INVALID, "tile linear: X and Y must be 16-byte aligned");
    CUtensorMap tm, tmy;
    if (!make_tmap_panels_f16(&tm, X, (uint64_t)T, (uint64_t)w->K, (uint64_t)w->K, kSlab, kKC / kPanel) ||
        !make_tmap_2d_f16(&tmy, Y, (uint64_t)T, (uint64_t)w->N, (uint64_t)w->N, 32, kUnitCols, 64))
        return fail(ET_ERR_CUDA, "tile linear: cuTensorMapEncodeTiled failed");
    using KernelFn = void (*)(CUtensorMap, CUtensorMap, GemmParams);
    // [mode][gelu]; GELU exists for the plain and the normalised-input epilogues
    static const KernelFn kernels[4][2] = {{tile_gemm_kernel<false, 0>, tile_gemm_kernel<true, 0>},
                                           {tile_gemm_kernel<false, 1>, tile_gemm_kernel<true, 1>},
                                           {tile_gemm_kernel<false, 2>, nullptr},
                                           {tile_gemm_kernel<false, 3>, nullptr}};
    static PerDeviceOnce once;
    const cudaError_t attr_err = once.run([] {
        cudaError_t e = cudaSuccess;
        for (int m = 0; m < 4 && e == cudaSuccess; ++m)
            for (int g = 0; g < 2 && e == cudaSuccess; ++g)
                if (kernels[m][g]) e = cudaFuncSetAttribute(kernels[m][g], cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        return e;
    });
    if (attr_err != cudaSuccess) return cuda_status(attr_err, "tile linear: shared memory opt-in");
    GemmParams p;
    p.dir = w->d_dir; p.stream = w->d_stream; p.Y = Y; p.bias = bias_dev ? bias_dev : w->d_bias;
    p.T = T; p.N = w->N; p.k_chunks = w->k_chunks; p.nb = w->nb;
    p.n_chunks = w->n_chunks;
    p.n_tiles = ((T + kSlab - 1) / kSlab) * w->n_chunks;
    p.stage_b_bytes = w->stage_b_bytes; p.nx = w->nx; p.nw = w->nw; p.a_slots = w->a_slots; p.gelu = gelu; p.err = w->d_err;
    p.prof = g_prof;
    for (size_t c = 0; c < w->h_first.size(); ++c) p.first[c] = w->h_first[c];
    const size_t smem = (size_t)w->nx * kXStageBytes + (size_t)w->nw * w->stage_b_bytes +
                        (size_t)kEpiWarps * kUnitBytes + sizeof(Shared) + 1024;
    // Packed for SM time (several batches in flight): a CTA takes several tiles in a row even when SMs are free,
    // so that set-up and pipeline fill are paid once and the next tile's loads run under an epilogue.
    dim3 grid(std::min((p.n_tiles + w->tiles_per_cta - 1) / w->tiles_per_cta, sm_count()));
    const int mode = fusion ? fusion->mode : 0;
    if (mode < 0 || mode > 3 || !kernels[mode][gelu ? 1 : 0]) return fail(ET_ERR_INVALID, "tile linear: no kernel for this epilogue");
    if (mode) {
        p.fz = *fusion;
        p.fz.bias_f32 = w->d_bias_f32;
        if (mode == 1) {
            if (!w->d_colc || !w->d_cold || !p.fz.stats_in || p.fz.np_in <= 0) return fail(ET_ERR_INVALID, "tile linear: weight not folded for a normalised input");
            p.fz.colc = w->d_colc;
            p.fz.cold = w->d_cold;
            p.fz.inv_d_in = 1.0f / (float)w->K;
        } else {
            if (!p.fz.resid || !p.fz.stats_out || p.fz.np_out != kEpiPerQuarter * w->n_chunks) return fail(ET_ERR_INVALID, "tile linear: residual epilogue needs a residual and 4 x chunks partial slots");
            if (mode == 3 && (!p.fz.stats_src || p.fz.np_src <= 0 || !p.fz.gamma_s || !p.fz.beta_s)) return fail(ET_ERR_INVALID, "tile linear: lazy residual needs its statistics and LayerNorm vectors");
            p.fz.inv_d_src = 1.0f / (float)w->N;
        }
    } else {
        p.fz = GemmFusion{};
    }
    const cudaError_t le = launch_pdl(kernels[mode][gelu ? 1 : 0], grid, dim3(kThreads), smem, st, tm, tmy, p);
    if (le != cudaSuccess) return cuda_status(le, "tile linear launch");
    return cuda_status(cudaGetLastError(), "tile linear launch");
}

int tile_weight_out_feat(const TileWeight* w) { return w->N; }
int tile_weight_chunks(const TileWeight* w) { return w->n_chunks; }
int tile_weight_stat_slots(const TileWeight* w) { return kEpiPerQuarter * w->n_chunks; }

// The weight with a LayerNorm folded in: tile values multiplied by gamma of their input feature (rounded to fp16
// again), c_n summed over those rounded values so that the epilogue's correction matches the products exactly.
int tile_weight_fold(TileWeight** out, const TileWeight* w, const half* gamma, const half* beta) {
    if (!out || !w || !gamma || !beta) return fail(ET_ERR_INVALID, "tile weight fold: null pointer");
    *out = nullptr;
    const int NBR = w->N / 16;
    std::vector<half> data(w->h_data.size());
    std::vector<double> c((size_t)w->N, 0.0), d((size_t)w->N, 0.0);
    for (int r = 0; r < NBR; ++r)
        for (int i = w->h_row_ptr[r]; i < w->h_row_ptr[r + 1]; ++i) {
            const int k0 = w->h_row_offset[i];
            for (int n = 0; n < 16; ++n)
                for (int k = 0; k < 16; ++k) {
                    const size_t at = (size_t)i * 256 + n * 16 + k;
                    const float wv = __half2float(w->h_data[at]);
                    const half folded = __float2half(wv * __half2float(gamma[k0 + k]));
                    data[at] = folded;
                    c[16 * r + n] += (double)__half2float(folded);
                    d[16 * r + n] += (double)wv * (double)__half2float(beta[k0 + k]);
                }
        }
    TileWeight* f = nullptr;
    int rc = tile_weight_pack(&f, w->K, w->N, w->size_hint, w->ntile, data.data(), w->h_row_ptr.data(), w->h_row_offset.data(),
                              w->h_bias.data(), 0);
    if (rc) return rc;
    std::vector<float> cf((size_t)w->N), df((size_t)w->N);
    for (int n = 0; n < w->N; ++n) {
        cf[n] = (float)c[n];
        df[n] = (float)(d[n] + (double)__half2float(w->h_bias[n]));
    }
    if (cudaMalloc(&f->d_colc, cf.size() * sizeof(float)) != cudaSuccess || cudaMalloc(&f->d_cold, df.size() * sizeof(float)) != cudaSuccess) {
        tile_weight_free(f);
        return fail(ET_ERR_CUDA, "tile weight fold: cudaMalloc failed");
    }
    cudaMemcpy(f->d_colc, cf.data(), cf.size() * sizeof(float), cudaMemcpyHostToDevice);
    cudaMemcpy(f->d_cold, df.data(), df.size() * sizeof(float), cudaMemcpyHostToDevice);
    *out = f;
    return ET_OK;
}

int tile_weight_error(const TileWeight* w, int* code) {
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, w->d_err, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_status(e, "tile weight error read");
    *code = v;
    if (v) cudaMemset(w->d_err, 0, sizeof(int));
    return ET_OK;
}

void tile_weight_info(const TileWeight* w, int* info) {
    info[0] = w->nb; info[1] = w->n_chunks; info[2] = w->k_chunks; info[3] = w->nx;   // activation slots (the weight ring has w->nw, chosen from the same memory)
    info[4] = w->stage_b_bytes; info[5] = (int)std::min<size_t>(w->stream_bytes, 0x7fffffff);
}

// ---- launcher-level entry with device-resident BSR arrays: packed form cached per weight ----
namespace {
std::mutex g_cache_mu;
std::map<std::tuple<const void*, const void*, const void*, int, int>, TileWeight*> g_cache;
}

int tile_spmm_raw(half* Y, const half* X, const int* row_ptr, const int* row_offset, const half* data,
                  int M, int N, int K, const half* bias, int gelu, cudaStream_t st) {
    if (!row_ptr || !bias) return fail(ET_ERR_INVALID, "tile spmm: null pointer");
    if (N <= 0 || K <= 0 || N % 16 || K % 16) return fail(ET_ERR_INVALID, "tile spmm: N and K must be positive multiples of 16");
    TileWeight* w = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_cache_mu);
        auto key = std::make_tuple((const void*)row_ptr, (const void*)row_offset, (const void*)data, N, K);
        auto it = g_cache.find(key);
        if (it == g_cache.end()) {
            std::vector<int> rp(N / 16 + 1);
            if (cudaMemcpy(rp.data(), row_ptr, rp.size() * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
                return fail(ET_ERR_CUDA, "tile spmm: cannot read row_ptr");
            const long ntile = rp.back();
            if (ntile < 0 || ntile > (long)(N / 16) * (K / 16) * 4) return fail(ET_ERR_INVALID, "tile spmm: implausible tile count");
            std::vector<int> ro(ntile);
            std::vector<half> dt((size_t)ntile * 256);
            if (ntile) {
                cudaMemcpy(ro.data(), row_offset, ntile * sizeof(int), cudaMemcpyDeviceToHost);
                cudaMemcpy(dt.data(), data, dt.size() * sizeof(half), cudaMemcpyDeviceToHost);
            }
            int rc = tile_weight_pack(&w, K, N, M, ntile, dt.data(), rp.data(), ro.data(), nullptr, 0);
            if (rc) return rc;
            g_cache[key] = w;
        } else {
            w = it->second;
        }
    }
    // the caller's bias is a kernel argument: nothing of the call is kept in the cached weight
    return tile_linear_run(w, Y, X, M, gelu, st, bias);
}

void tile_spmm_cache_clear() {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    for (auto& kv : g_cache) tile_weight_free(kv.second);
    g_cache.clear();
}

}  // namespace et
