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
//   * A ring of R slots, each one shared-memory stage plus one TMEM A slot, with one barrier hop per role
//     and chunk: producer waits slot_free -> TMA; mover waits full -> tcgen05.cp -> commit a_ready;
//     issuers wait a_ready -> UMMAs -> commit slot_free. (A wait that follows the same thread's
//     tcgen05.commit costs a few hundred clocks, so hops per chunk are what the loop time is made of.)
//   * Epilogue: tcgen05.ld, + bias, optional GELU, fp16, staged in shared memory in 128-byte-swizzled
//     64-column panels and written with TMA stores (rows beyond T and columns beyond N are clipped).
// Every mbarrier wait is bounded; a wait that gives up records a code in the error word, the CTA
// stops issuing, frees its tensor memory and returns.
#include <algorithm>
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
constexpr int kMaxSlots = 4;
constexpr int kIssuers = 8;         // UMMA-issuing warps
constexpr int kMovers = 2;          // tcgen05.cp-issuing warps, alternating chunks
constexpr int kFirstIssuer = 1 + kMovers;
constexpr int kThreads = 32 * (1 + kMovers + kIssuers);
constexpr int kDirInParams = 32;    // directory entries of each chunk's first block travel as kernel parameters
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
    int T, N, k_chunks, n_chunks, n_tiles, nb, stage_b_bytes, slots, a_slots, panel_bufs, gelu;
    int* err;
    uint2 first[kDirInParams];   // dir[chunk][0] for chunk < kDirInParams: no global load before the first TMA
    long long* prof;         // optional per-role clock64 stamps of CTA (0,0) (ET_GEMM_PROFILE builds only)
};

// Timing experiments (never in the shipped library): -DET_GEMM_EXPERIMENT=<mask> removes one stage's work
// while keeping every barrier hop, to see what a chunk's time is made of. 1: no weight copy, 2: no UMMAs,
// 4: no tcgen05.cp, 8: no activation TMA.
#ifndef ET_GEMM_EXPERIMENT
#define ET_GEMM_EXPERIMENT 0
#endif

#ifdef ET_GEMM_PROFILE
#define ET_STAMP(slot) do { if (p.prof && blockIdx.x == 0 && blockIdx.y == 0) p.prof[(slot)] = clock64(); } while (0)
#else
#define ET_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}"
                 : "=r"(pred));
    return pred != 0;
}
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
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
    return 0.5f * x * (1.0f + tanh_fast(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

struct Shared {
    uint64_t full[kMaxSlots];       // stage filled: two activation panels + the weight block (TMA)
    uint64_t a_ready[kMaxSlots];    // the chunk's activations are in their tensor-memory slot (mover commit)
    uint64_t slot_free[kMaxSlots];  // every issuer's UMMAs on the stage have completed (8 commits)
    uint64_t acc_done;              // 8 issuer commits after a tile's last chunk
    uint32_t tmem_base;
    volatile int abort;         // any role gave up: everybody winds down
    volatile int issuer_abort;  // written by issuer warps only, before a tile's last named barrier, and read
                                // after it: all eight warps leave the tile loop at the same tile
    __align__(16) half bias[kMaxNB * 16];  // the current tile's bias
};

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void tma_store_wait_read_1() {
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}

// Persistent: CTA c processes tiles c, c + gridDim.x, ... (tile = slab * n_chunks + chunk, so CTAs that run
// together share activations in L2). The slot ring runs on across tiles: while the issuer warps convert and
// store one tile, the producer and the movers already stage the first chunks of the next.
__global__ void __launch_bounds__(kThreads, 1)
tile_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int slot_bytes = kXStageBytes + p.stage_b_bytes;   // multiple of 1024
    uint8_t* panels = smem + (size_t)p.slots * slot_bytes;   // one or two 16 KB output panels
    Shared* sh = reinterpret_cast<Shared*>(panels + p.panel_bufs * kPanelBytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Two rings with one chunk counter: R shared-memory stages (activations + weight block; a stage is free
    // once the chunk's UMMAs have completed, because they read the weights from it) and RA <= R tensor-memory
    // slots for the A operand. A chunk's tensor-memory slot is free when the chunk RA before it is done, which
    // the movers read from the same slot_free barriers with a lag.
    const int R = p.slots, RA = p.a_slots;
    const int G = gridDim.x;
    const uint32_t a_col0 = 512u - (uint32_t)(RA * kSlotCols);
    const int my_tiles = (p.n_tiles - (int)blockIdx.x + G - 1) / G;
    if (tid == 0) ET_STAMP(0);
    pdl_launch_dependents();   // the next kernel may set itself up on idle SMs while this one runs

    if (warp == 0) {
        // ---------------- producer warp: lane 0 issues the copies, lane 1 polls slot_free (a wait by the thread
        // that has just issued a bulk copy costs several hundred clocks)
        {
            // one barrier per lane
            if (lane < kMaxSlots) mbar_init(&sh->full[lane], 1);
            else if (lane < 2 * kMaxSlots) mbar_init(&sh->a_ready[lane - kMaxSlots], 1);
            else if (lane < 3 * kMaxSlots) mbar_init(&sh->slot_free[lane - 2 * kMaxSlots], kIssuers);
            else if (lane == 3 * kMaxSlots) mbar_init(&sh->acc_done, kIssuers);
            if (lane <= 3 * kMaxSlots) fence_mbar_init();
            if (lane == 0) {
                sh->abort = 0;
                sh->issuer_abort = 0;
            }
        }
        __syncwarp();
        named_barrier_arrive(2, kThreads);   // barriers are initialised: release the other warps
        if (lane == 0) ET_STAMP(8);
        // Everything above touched only this kernel's own resources. The activations may still be in the making:
        // wait for the preceding kernels before the first copy (lane 0 issues them all).
        if (lane == 0) pdl_wait();
        int issued = 0, r = 0;
        uint32_t ph = 0;
        bool alive = true;
        for (int tl = 0; tl < my_tiles && alive; ++tl) {
            const int tile = (int)blockIdx.x + tl * G;
            const int slab = tile / p.n_chunks, chunk = tile - slab * p.n_chunks;
            const uint2* gdir = p.dir + (size_t)chunk * p.k_chunks;
            // directory entries: the first one of the first tile comes from the kernel parameters, the others are
            // fetched one chunk ahead
            uint2 dnext = (tl == 0 && chunk < kDirInParams) ? p.first[chunk] : (lane == 0 ? __ldg(gdir) : make_uint2(0, 0));
            for (int kc = 0; kc < p.k_chunks; ++kc) {
                const uint2 d = dnext;
                if (lane == 0 && kc + 1 < p.k_chunks) dnext = __ldg(gdir + kc + 1);
                int go = 1;
                if (lane == 1) go = (!sh->abort && mbar_wait(&sh->slot_free[r], ph ^ 1u)) ? 1 : 0;
                go = __shfl_sync(0xffffffffu, go, 1);
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
                    uint8_t* st = smem + (size_t)r * slot_bytes;
                    const uint32_t bbytes = d.y * 16u;
                    mbar_expect_tx(&sh->full[r], kXStageBytes + bbytes);
                    tma_load_3d(st, &tmX, 0, slab * kSlab, kc * (kKC / kPanel), &sh->full[r]);   // both panels, one op
                    bulk_load(st + kXStageBytes, p.stream + (size_t)d.x * 16u, bbytes, &sh->full[r]);
                    if (issued < 64) ET_STAMP(100 + issued);
                }
                ++issued;
                if (++r == R) { r = 0; ph ^= 1u; }
            }
        }
        // Leaving early: wait (bounded) for the copies still in flight before the CTA exits.
        if (lane == 1 && sh->abort)
            for (int kk = issued > R ? issued - R : 0; kk < issued; ++kk)
                mbar_wait(&sh->full[kk % R], (uint32_t)(kk / R) & 1u);
    } else {
        if (warp == 1) {
            tmem_alloc(&sh->tmem_base, 512);
            tmem_relinquish();
        }
        tc_fence_before();
        named_barrier_sync(1, kThreads - 32);   // all but the producer: the tensor-memory base is visible
        tc_fence_after();
        const uint32_t tmem = sh->tmem_base;
        // Accumulators start at zero: block-rows without tiles are legal and every UMMA accumulates. (After
        // each tile the epilogue clears them again.)
        if (warp >= kFirstIssuer) {
            const int w = warp - kFirstIssuer;
            const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
            for (int br = (w >> 2); br < p.nb; br += 2) tmem_st16_zero(tmem + lane_base + br * 16);
            tmem_st_wait();
        }
        tc_fence_before();
        named_barrier_sync(2, kThreads);        // + the producer's arrive: mbarriers are initialised
        tc_fence_after();
        if (tid == 32) ET_STAMP(2);
        const int n_items = my_tiles * p.k_chunks;

        if (warp < kFirstIssuer) {
            // ---------------- movers: shared memory -> tensor memory copy of the A operand. Two warps take
            // alternate chunks; lane 1 polls, lane 0 issues and commits.
            const int m = warp - 1;
            int r = m % R, a = m % RA;
            uint32_t ph = (uint32_t)(m / R) & 1u;
            for (int it = m; it < n_items; it += kMovers) {
                if (sh->abort) break;
                int got = 1;
                if (lane == 1) {
                    got = mbar_wait(&sh->full[r], ph);
                    if (got && it >= RA) {   // the tensor-memory slot: chunk it - RA must be done
                        const int prev = it - RA;
                        got = mbar_wait(&sh->slot_free[prev % R], (uint32_t)(prev / R) & 1u);
                    }
                }
                got = __shfl_sync(0xffffffffu, got, 1);
                if (lane == 0 && it < 64) ET_STAMP(700 + it);
                if (!got) {
                    if (lane == 0) atomicExch(p.err, 12);
                    sh->abort = 1;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t xa = smem_u32(smem + (size_t)r * slot_bytes);
                    const uint32_t ta = tmem + a_col0 + a * kSlotCols;
#pragma unroll
                    for (int sl = 0; sl < kSlices; ++sl)
                        tc_cp_128x256b(ta + sl * 8,
                                       make_smem_desc(xa + (sl >> 2) * kPanelBytes + (sl & 3) * 32, 16, 1024, 2));
                    umma_commit(&sh->a_ready[a]);
                    if (it < 64) ET_STAMP(300 + it);
                }
                __syncwarp();
                r += kMovers;
                while (r >= R) { r -= R; ph ^= 1u; }
                a = (a + kMovers) % RA;
            }
        } else {
            // ---------------- issuers: one UMMA per kept tile, A from tensor memory; then the tile's epilogue
            const int w = warp - kFirstIssuer;
            const int q = warp & 3;
            const int row = q * 32 + lane;                 // row of the slab = TMEM lane
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            // B tile descriptor: no swizzle, 128 B between core matrices along K, 256 B along N.
            const uint64_t b_desc0 = make_smem_desc(0, 128, 256, 0);
            bool ok = true;
            int r = 0, a = 0;
            uint32_t pha = 0;
            int stores = 0;   // output panels handed to TMA so far (panel buffers alternate)
            for (int tl = 0; tl < my_tiles; ++tl) {
                const int tile = (int)blockIdx.x + tl * G;
                const int slab = tile / p.n_chunks, chunk = tile - slab * p.n_chunks;
                // this tile's bias (read by the epilogue; the barrier below also orders the accumulator clear)
                {
                    const int col0 = chunk * p.nb * 16;
                    for (int i = tid - 32 * kFirstIssuer; i < p.nb * 16; i += 32 * kIssuers)
                        sh->bias[i] = (col0 + i < p.N) ? p.bias[col0 + i] : __float2half(0.f);
                }
                named_barrier_sync(3, 32 * kIssuers);
                for (int kc = 0; kc < p.k_chunks && ok; ++kc) {
                    if (sh->abort) {
                        sh->issuer_abort = 1;
                        ok = false;
                        break;
                    }
                    // a_ready implies full: the mover waited for the slot's TMA before copying. Lane 1 polls.
                    int got = 1;
                    if (lane == 1) {
                        got = mbar_wait(&sh->a_ready[a], pha);
                        if (w == 0 && tl * p.k_chunks + kc < 64) ET_STAMP(500 + tl * p.k_chunks + kc);
                    }
                    got = __shfl_sync(0xffffffffu, got, 1);
                    if (!got) {
                        if (lane == 0) atomicExch(p.err, 13);
                        sh->abort = 1;
                        sh->issuer_abort = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint8_t* blk = smem + (size_t)r * slot_bytes + kXStageBytes;
                    const uint32_t hw = reinterpret_cast<const uint32_t*>(blk)[w];
                    const int e0 = hw & 0xffff, ne = hw >> 16;
                    const uint32_t n_entries = reinterpret_cast<const uint32_t*>(blk)[8];
                    const uint4* ent = reinterpret_cast<const uint4*>(blk + kHeaderBytes) + e0;
                    const uint32_t tiles16 = (smem_u32(blk) + kHeaderBytes + n_entries * 16u) >> 4;
                    const uint32_t abuf = tmem + a_col0 + a * kSlotCols;
#pragma unroll 4
                    for (int i = 0; i < ne; ++i) {
                        const uint4 e = ent[i];
                        if (!(ET_GEMM_EXPERIMENT & 2) && elect_one())
                            umma_f16_ts(tmem + e.z, abuf + e.y, b_desc0 | (uint64_t)((tiles16 + e.x) & 0x3fff), e.w, 1u);
                    }
                    if (elect_one()) umma_commit(&sh->slot_free[r]);
                    if (w == 0 && lane == 0 && tl * p.k_chunks + kc < 64) ET_STAMP(600 + tl * p.k_chunks + kc);
                    __syncwarp();
                    if (++r == R) r = 0;
                    if (++a == RA) { a = 0; pha ^= 1u; }
                }
                if (elect_one()) umma_commit(&sh->acc_done);
                __syncwarp();

                // ---------------- epilogue: TMEM -> registers -> bias / GELU -> fp16 -> swizzled panel -> TMA store
                if (ok) {
                    int done = 1;
                    if (lane == 1) done = mbar_wait(&sh->acc_done, (uint32_t)tl & 1u);
                    done = __shfl_sync(0xffffffffu, done, 1);
                    if (!done) {
                        if (lane == 0) atomicExch(p.err, 14);
                        sh->abort = 1;
                        sh->issuer_abort = 1;
                        ok = false;
                    }
                }
                tc_fence_after();
                if (w == 0 && lane == 0 && tl < 16) ET_STAMP(1400 + tl * 16);
                const int npanels = (p.nb + 3) >> 2;
                for (int pi = 0; pi < npanels; ++pi, ++stores) {
                    uint8_t* pbuf = panels + (size_t)(stores & (p.panel_bufs - 1)) * kPanelBytes;
                    const int lb = pi * 4 + (w >> 2), lb2 = lb + 2;
                    uint4 ov[2][2];
                    const bool has1 = ok && lb < p.nb, has2 = ok && lb2 < p.nb;
                    if (has1) {
                        uint32_t acc[2][16];
                        tmem_ld16(tmem + lane_base + lb * 16, acc[0]);
                        if (has2) tmem_ld16(tmem + lane_base + lb2 * 16, acc[1]);
                        tmem_ld_wait();
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            if (u == 1 && !has2) break;
                            const int l = u ? lb2 : lb;
                            const half2* bh = reinterpret_cast<const half2*>(sh->bias + l * 16);
                            half2* oh = reinterpret_cast<half2*>(ov[u]);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float2 bb = __half22float2(bh[i]);
                                float v0 = __uint_as_float(acc[u][2 * i]) + bb.x;
                                float v1 = __uint_as_float(acc[u][2 * i + 1]) + bb.y;
                                if (p.gelu) {
                                    v0 = gelu_tanh(v0);
                                    v1 = gelu_tanh(v1);
                                }
                                oh[i] = __floats2half2_rn(v0, v1);
                            }
                        }
                    }
                    // the buffer was handed to TMA one or two panels ago: that store must have finished reading it
                    if (w == 0 && lane == 0) {
                        if (p.panel_bufs == 2) tma_store_wait_read_1();
                        else tma_store_wait_read();
                    }
                    named_barrier_sync(3, 32 * kIssuers);
                    if (has1) {
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            if (u == 1 && !has2) break;
                            const int l = u ? lb2 : lb;
                            // 16-byte chunks 2*(l%4) and 2*(l%4)+1 of the row, 128-byte swizzle
                            uint8_t* prow = pbuf + row * 128;
                            const int c0 = (l & 3) * 2;
                            *reinterpret_cast<uint4*>(prow + (((c0) ^ (row & 7)) << 4)) = ov[u][0];
                            *reinterpret_cast<uint4*>(prow + (((c0 + 1) ^ (row & 7)) << 4)) = ov[u][1];
                        }
                        fence_proxy_async_smem();
                    }
                    named_barrier_sync(3, 32 * kIssuers);   // the panel is complete
                    if (w == 0 && lane == 0) {
                        const int col = chunk * p.nb * 16 + pi * kPanel;
                        if (!sh->abort && col < p.N) tma_store_2d(&tmY, pbuf, col, slab * kSlab);
                        tma_store_commit();
                        if (tl < 16 && pi < 14) ET_STAMP(1400 + tl * 16 + 1 + pi);
                    }
                }
                // clear the accumulators for the next tile (each warp its lane quarter and column half)
                if (tl + 1 < my_tiles) {
                    for (int br = (w >> 2); br < p.nb; br += 2) tmem_st16_zero(tmem + lane_base + br * 16);
                    tmem_st_wait();
                    tc_fence_before();
                }
                if (w == 0 && lane == 0 && tl < 16) ET_STAMP(1400 + tl * 16 + 15);
                if (sh->issuer_abort) break;
            }
            if (w == 0 && lane == 0) tma_store_wait_read();   // shared memory may go once the stores have read it
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) ET_STAMP(4);
    if (warp == 1) tmem_dealloc(sh->tmem_base, 512);
}

}  // namespace

// --------------------------------------------------------------------------------- host side

struct TileWeight {
    int K = 0, N = 0, nb = 0, n_chunks = 0, k_chunks = 0, stage_b_bytes = 0, slots = 0, a_slots = 0, panel_bufs = 1;
    long ntile = 0;
    int size_hint = 0;
    // the caller's arrays, kept so that weights can be concatenated (Q|K|V in one launch) and re-packed
    std::vector<int> h_row_ptr, h_row_offset;
    std::vector<half> h_data, h_bias;
    std::vector<uint2> h_first;   // directory entry of each chunk's first block
    uint2* d_dir = nullptr;
    uint8_t* d_stream = nullptr;
    half* d_bias = nullptr;
    int* d_err = nullptr;
    size_t stream_bytes = 0;
};

// Block-rows per CTA from a model of the persistent kernel: a slot of the ring takes about 2300 clocks to go
// round (TMA, tcgen05.cp, UMMAs, commit, poll), R slots are in flight, a chunk cannot be faster than its UMMAs
// (~10 clocks each with eight issuing warps), and a tile ends with ~800 clocks of epilogue per 64-column panel.
struct RingShape { int stages, a_slots, panel_bufs; };
static RingShape ring_shape(int nb, int stage_b_bytes) {
    const int slot = kXStageBytes + stage_b_bytes;
    const int avail = kSmemMax - 1024 - (int)sizeof(Shared);
    RingShape s;
    s.stages = std::min(kMaxSlots, (avail - kPanelBytes) / slot);
    s.panel_bufs = avail - s.stages * slot >= 2 * kPanelBytes ? 2 : 1;
    s.a_slots = std::min(s.stages, (512 - nb * 16) / kSlotCols);
    return s;
}
static int choose_nb(int n_block_rows, int k_chunks, int size_hint, double density) {
    const int slabs = std::max(1, (size_hint + kSlab - 1) / kSlab);
    const int sms = std::max(1, sm_count());
    double best = 0;
    int best_nb = 0;
    for (int nb : {24, 20, 16, 12, 8}) {
        // chunks other than a single one must cover whole 64-column output panels (nb % 4 == 0)
        const int nbe = n_block_rows <= nb ? std::max(n_block_rows, 1) : nb;
        if (nbe > kMaxNB) continue;
        const double tiles_per_chunk = nbe * kSlices * density;
        const int stage_b = (int)((kHeaderBytes + tiles_per_chunk * 1.5 * 528.0 + 1023) / 1024) * 1024;   // worst block ~1.5x mean
        const RingShape rs = ring_shape(nbe, stage_b);
        if (rs.stages < 2 || rs.a_slots < 1) continue;
        const long tiles = (long)slabs * ((n_block_rows + nbe - 1) / nbe);
        const double per_cta = (double)((tiles + sms - 1) / sms);
        // stage cycle, tensor-memory slot cycle, UMMA issue, and the SM's share of L2 bandwidth (~64 B/clock)
        const double t_chunk = std::max({2200.0 / rs.stages, 1100.0 / rs.a_slots, 10.0 * tiles_per_chunk,
                                         (kXStageBytes + tiles_per_chunk * 528.0) / 64.0});
        const double t_tile = k_chunks * t_chunk + 800.0 * ((nbe + 3) / 4) + 500.0;
        const double cost = per_cta * t_tile + 3000.0;
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
        w->slots = rs.stages; w->a_slots = rs.a_slots; w->panel_bufs = rs.panel_bufs;
    }
    if (w->slots < 2) { delete w; return fail(ET_ERR_UNSUPPORTED, "tile weight: weight block exceeds shared memory"); }
    w->stream_bytes = stream.size();

    cudaError_t e1 = cudaMalloc(&w->d_dir, dir.size() * sizeof(uint2));
    cudaError_t e2 = cudaMalloc(&w->d_stream, std::max<size_t>(stream.size(), 16));
    cudaError_t e3 = cudaMalloc(&w->d_bias, (size_t)N * sizeof(half));
    cudaError_t e4 = cudaMalloc(&w->d_err, sizeof(int));
    if (e1 || e2 || e3 || e4) { tile_weight_free(w); return fail(ET_ERR_CUDA, "tile weight: cudaMalloc failed"); }
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
    delete w;
}

int tile_weight_set_bias_device(TileWeight* w, const half* bias_dev, cudaStream_t st) {
    return cuda_status(cudaMemcpyAsync(w->d_bias, bias_dev, (size_t)w->N * sizeof(half), cudaMemcpyDeviceToDevice, st), "bias copy");
}

static long long* g_prof = nullptr;
void tile_gemm_set_profile_buffer(long long* dev_buf) { g_prof = dev_buf; }

int tile_linear_run(const TileWeight* w, half* Y, const half* X, int T, int gelu, cudaStream_t st) {
    if (!w || !Y || !X) return fail(ET_ERR_INVALID, "tile linear: null pointer");
    if (T < 0) return fail(ET_ERR_INVALID, "tile linear: negative token count");
    if (T == 0) return ET_OK;
    if (!aligned16(X) || !aligned16(Y)) return fail(ET_ERR_INVALID, "tile linear: X and Y must be 16-byte aligned");
    CUtensorMap tm, tmy;
    if (!make_tmap_panels_f16(&tm, X, (uint64_t)T, (uint64_t)w->K, (uint64_t)w->K, kSlab, kKC / kPanel) ||
        !make_tmap_2d_f16(&tmy, Y, (uint64_t)T, (uint64_t)w->N, (uint64_t)w->N, kSlab, kPanel, true))
        return fail(ET_ERR_CUDA, "tile linear: cuTensorMapEncodeTiled failed");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(tile_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
    });
    if (attr_err != cudaSuccess) return cuda_status(attr_err, "tile linear: shared memory opt-in");
    GemmParams p;
    p.dir = w->d_dir; p.stream = w->d_stream; p.Y = Y; p.bias = w->d_bias;
    p.T = T; p.N = w->N; p.k_chunks = w->k_chunks; p.nb = w->nb;
    p.n_chunks = w->n_chunks;
    p.n_tiles = ((T + kSlab - 1) / kSlab) * w->n_chunks;
    p.stage_b_bytes = w->stage_b_bytes; p.slots = w->slots; p.a_slots = w->a_slots; p.panel_bufs = w->panel_bufs; p.gelu = gelu; p.err = w->d_err;
    p.prof = g_prof;
    for (size_t c = 0; c < w->h_first.size(); ++c) p.first[c] = w->h_first[c];
    const size_t smem = (size_t)w->slots * (kXStageBytes + w->stage_b_bytes) + (size_t)w->panel_bufs * kPanelBytes + sizeof(Shared) + 1024;
    dim3 grid(std::min(p.n_tiles, sm_count()));
    const cudaError_t le = launch_pdl(tile_gemm_kernel, grid, dim3(kThreads), smem, st, tm, tmy, p);
    if (le != cudaSuccess) return cuda_status(le, "tile linear launch");
    return cuda_status(cudaGetLastError(), "tile linear launch");
}

int tile_weight_out_feat(const TileWeight* w) { return w->N; }

int tile_weight_error(const TileWeight* w, int* code) {
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, w->d_err, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_status(e, "tile weight error read");
    *code = v;
    if (v) cudaMemset(w->d_err, 0, sizeof(int));
    return ET_OK;
}

void tile_weight_info(const TileWeight* w, int* info) {
    info[0] = w->nb; info[1] = w->n_chunks; info[2] = w->k_chunks; info[3] = w->slots;
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
    int rc = tile_weight_set_bias_device(w, bias, st);
    if (rc) return rc;
    return tile_linear_run(w, Y, X, M, gelu, st);
}

void tile_spmm_cache_clear() {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    for (auto& kv : g_cache) tile_weight_free(kv.second);
    g_cache.clear();
}

}  // namespace et
