// Tile-sparse linear  Y[T x N] = X[T x K] . W^T + bias  (optional tanh-GELU), W in 16x16 tile-BSR.
// Replaces kernels/linear.cu:54-167 of the reference (both kernels and both launchers) and the
// weight side of encoder/Linear.h:4-46.
//
// sm_100a design (tcgen05 + TMEM + TMA), zero tiles are never touched:
//   * A CTA owns a slab of 128 tokens and a chunk of up to 24 output block-rows (16 features each).
//     Its fp32 accumulators live in tensor memory: 16 TMEM columns per block-row, 384 columns at most.
//   * The activations are the A operand and are read from tensor memory, not shared memory: X is
//     brought in by TMA (128-byte-swizzled 128 x 64 panels) and moved smem -> TMEM with tcgen05.cp
//     into one of four 32-column buffers. With A in TMEM a 128x16x16 UMMA no longer pays the
//     4 KB shared-memory read of A, which otherwise bounds small-N UMMAs to ~20 % of tensor peak.
//   * Every kept tile is one UMMA  D[128 x 16] += A[128 x 16] . tile^T  (B operand = the tile in
//     shared memory, canonical no-swizzle K-major layout). A single warp can only issue one UMMA per
//     ~55 clocks, so eight warps issue concurrently, each owning a disjoint set of block-rows.
//   * The weight is re-packed once, on the host, into a stream of blocks, one per (block-row chunk,
//     64-wide K chunk): a per-warp issue list followed by the tiles already in UMMA layout. One
//     cp.async.bulk brings a block into shared memory. The sparsity pattern is kept exactly.
//   * Epilogue: tcgen05.ld, + bias, optional GELU, fp16, 32 contiguous bytes per (row, block-row).
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
constexpr int kKC = 64;             // K elements per chunk = one 128-byte-swizzled panel
constexpr int kSlices = kKC / 16;   // UMMA K steps per chunk
constexpr int kMaxNB = 24;          // block-rows per CTA (384 accumulator columns)
constexpr int kABufs = 4;           // A buffers in tensor memory, 32 columns each
constexpr int kACol0 = 384;         // first A column
constexpr int kIssuers = 8;         // UMMA-issuing warps
constexpr int kThreads = 32 * (2 + kIssuers);
constexpr int kXStageBytes = kSlab * kKC * 2;  // 16 KB
constexpr int kHeaderBytes = 64;
constexpr int kMaxStages = 8;
constexpr int kSmemMax = 232448;    // 227 KB: the per-CTA opt-in limit of sm_100
constexpr int kMaxKChunks = 512;    // in_feat up to 32768

struct GemmParams {
    const uint2* dir;        // per (chunk, k-chunk): {offset, size} in 16-byte units
    const uint8_t* stream;   // packed blocks
    half* Y;
    const half* bias;
    int T, N, k_chunks, nb, stage_b_bytes, num_stages, gelu;
    int* err;
    long long* prof;         // optional per-role clock64 stamps of CTA (0,0) (ET_GEMM_PROFILE builds only)
};

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
    uint64_t full[kMaxStages];        // stage filled (TMA X panel + weight block)
    uint64_t stage_free[kMaxStages];  // 1 mover + 8 issuer commits
    uint64_t a_ready[kABufs];         // A buffer holds this chunk's activations
    uint64_t a_free[kABufs];          // 8 issuer commits
    uint64_t acc_done;                // 8 issuer commits after the last chunk
    uint32_t tmem_base;
    volatile int abort;
    uint2 dir[kMaxKChunks];           // this CTA's row of the block directory
};

__global__ void __launch_bounds__(kThreads, 1)
tile_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int stage_bytes = kXStageBytes + p.stage_b_bytes;  // multiple of 1024
    Shared* sh = reinterpret_cast<Shared*>(smem + (size_t)p.num_stages * stage_bytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slab = blockIdx.x, chunk = blockIdx.y;
    const int S = p.num_stages;
    if (tid == 0) ET_STAMP(0);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->stage_free[s], 1 + kIssuers);
        }
        for (int j = 0; j < kABufs; ++j) {
            mbar_init(&sh->a_ready[j], 1);
            mbar_init(&sh->a_free[j], kIssuers);
        }
        mbar_init(&sh->acc_done, kIssuers);
        sh->abort = 0;
        fence_mbar_init();
        prefetch_tmap(&tmX);
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    } else if (warp == 0) {
        const uint2* gdir = p.dir + (size_t)chunk * p.k_chunks;
        for (int i = lane; i < p.k_chunks; i += 32) sh->dir[i] = __ldg(gdir + i);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    if (tid == 0) ET_STAMP(1);

    // Accumulators start at zero: block-rows without tiles are legal and every UMMA accumulates.
    if (warp >= 2) {
        const int w = warp - 2;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        for (int br = (w >> 2); br < p.nb; br += 2) tmem_st16_zero(tmem + lane_base + br * 16);
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (tid == 0) ET_STAMP(2);

    if (warp == 0) {
        // ---------------- producer: TMA activations + bulk copy of the weight block
        if (lane == 0) {
            int issued = 0;
            for (int kc = 0; kc < p.k_chunks; ++kc) {
                const int s = kc % S;
                const uint32_t ph = (uint32_t)(kc / S) & 1u;
                const uint2 d = sh->dir[kc];
                if (sh->abort) break;
                const bool free_ok = mbar_wait(&sh->stage_free[s], ph ^ 1u);
                ET_STAMP(900 + kc);
                if (!free_ok) {
                    atomicExch(p.err, 11);
                    sh->abort = 1;
                    break;
                }
                uint8_t* st = smem + (size_t)s * stage_bytes;
                const uint32_t bbytes = d.y * 16u;
                mbar_expect_tx(&sh->full[s], kXStageBytes + bbytes);
                ET_STAMP(1000 + kc);
                tma_load_2d(st, &tmX, kc * kKC, slab * kSlab, &sh->full[s]);
                ET_STAMP(1100 + kc);
                bulk_load(st + kXStageBytes, p.stream + (size_t)d.x * 16u, bbytes, &sh->full[s]);
                ET_STAMP(100 + kc);
                ++issued;
            }
            // Leaving early: wait (bounded) for the copies still in flight before the CTA exits.
            if (sh->abort)
                for (int kk = issued > S ? issued - S : 0; kk < issued; ++kk)
                    mbar_wait(&sh->full[kk % S], (uint32_t)(kk / S) & 1u);
        }
    } else if (warp == 1) {
        // ---------------- mover: shared memory -> tensor memory copy of the A operand
        if (lane == 0) {
            for (int kc = 0; kc < p.k_chunks; ++kc) {
                const int s = kc % S, j = kc % kABufs;
                if (sh->abort) break;
                bool got = mbar_wait(&sh->full[s], (uint32_t)(kc / S) & 1u);
                ET_STAMP(700 + kc);
                got = got && mbar_wait(&sh->a_free[j], ((uint32_t)(kc / kABufs) & 1u) ^ 1u);
                ET_STAMP(800 + kc);
                if (!got) {
                    atomicExch(p.err, 12);
                    sh->abort = 1;
                    break;
                }
                tc_fence_after();
                ET_STAMP(200 + kc);
                const uint32_t xa = smem_u32(smem + (size_t)s * stage_bytes);
#pragma unroll
                for (int sl = 0; sl < kSlices; ++sl)
                    tc_cp_128x256b(tmem + kACol0 + j * 32 + sl * 8,
                                   make_smem_desc(xa + sl * 32, 16, 1024, 2));
                umma_commit(&sh->a_ready[j]);
                umma_commit(&sh->stage_free[s]);
                ET_STAMP(300 + kc);
            }
        }
    } else {
        // ---------------- issuers: one UMMA per kept tile, A from tensor memory
        const int w = warp - 2;
        // B tile descriptor: no swizzle, 128 B between core matrices along K, 256 B along N.
        const uint64_t b_desc0 = make_smem_desc(0, 128, 256, 0);
        bool ok = true;
        for (int kc = 0; kc < p.k_chunks && ok; ++kc) {
            const int s = kc % S, j = kc % kABufs;
            if (sh->abort) { ok = false; break; }
            // one lane polls; 256 threads spinning on the same mbarrier words slow every other
            // barrier operation of the CTA (TMA completion included)
            int got = 1;
            if (lane == 0) {
                got = mbar_wait(&sh->full[s], (uint32_t)(kc / S) & 1u);
                if (w == 0) ET_STAMP(400 + kc);
                got = got && mbar_wait(&sh->a_ready[j], (uint32_t)(kc / kABufs) & 1u);
                if (w == 0) ET_STAMP(500 + kc);
            }
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) {
                if (lane == 0) atomicExch(p.err, 13);
                sh->abort = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            const uint8_t* blk = smem + (size_t)s * stage_bytes + kXStageBytes;
            const uint32_t hw = reinterpret_cast<const uint32_t*>(blk)[w];
            const int e0 = hw & 0xffff, ne = hw >> 16;
            const uint32_t n_entries = reinterpret_cast<const uint32_t*>(blk)[8];
            const uint4* ent = reinterpret_cast<const uint4*>(blk + kHeaderBytes) + e0;
            const uint32_t tiles16 = (smem_u32(blk) + kHeaderBytes + n_entries * 16u) >> 4;
            const uint32_t abuf = tmem + kACol0 + j * 32;
#pragma unroll 4
            for (int i = 0; i < ne; ++i) {
                const uint4 e = ent[i];
                if (elect_one())
                    umma_f16_ts(tmem + e.z, abuf + e.y,
                                b_desc0 | (uint64_t)((tiles16 + e.x) & 0x3fff), e.w, 1u);
            }
            if (elect_one()) {
                umma_commit(&sh->stage_free[s]);
                umma_commit(&sh->a_free[j]);
            }
            if (w == 0 && lane == 0) ET_STAMP(600 + kc);
            __syncwarp();
        }
        if (elect_one()) umma_commit(&sh->acc_done);
        __syncwarp();

        // ---------------- epilogue: TMEM -> registers -> bias / GELU -> fp16 -> global
        if (ok) {
            int done = 1;
            if (lane == 0) done = mbar_wait(&sh->acc_done, 0);
            done = __shfl_sync(0xffffffffu, done, 0);
            if (!done) {
                if (lane == 0) atomicExch(p.err, 14);
                ok = false;
            }
        }
        tc_fence_after();
        if (w == 0 && lane == 0) ET_STAMP(3);
        if (ok) {
            const int q = warp & 3;
            const int row = slab * kSlab + q * 32 + lane;
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            for (int lb = (w >> 2); lb < p.nb; lb += 2) {
                const int col = (chunk * p.nb + lb) * 16;
                if (col >= p.N) break;
                uint32_t r[16];
                tmem_ld16(tmem + lane_base + lb * 16, r);
                tmem_ld_wait();
                if (row < p.T) {
                    const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + col);
                    uint4 bv[2] = {__ldg(b4), __ldg(b4 + 1)};
                    const half2* bh = reinterpret_cast<const half2*>(bv);
                    uint4 ov[2];
                    half2* oh = reinterpret_cast<half2*>(ov);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float2 bb = __half22float2(bh[i]);
                        float v0 = __uint_as_float(r[2 * i]) + bb.x;
                        float v1 = __uint_as_float(r[2 * i + 1]) + bb.y;
                        if (p.gelu) {
                            v0 = gelu_tanh(v0);
                            v1 = gelu_tanh(v1);
                        }
                        oh[i] = __floats2half2_rn(v0, v1);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.Y + (size_t)row * p.N + col);
                    dst[0] = ov[0];
                    dst[1] = ov[1];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) ET_STAMP(4);
    if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace

// --------------------------------------------------------------------------------- host side

struct TileWeight {
    int K = 0, N = 0, nb = 0, n_chunks = 0, k_chunks = 0, stage_b_bytes = 0, num_stages = 0;
    long ntile = 0;
    uint2* d_dir = nullptr;
    uint8_t* d_stream = nullptr;
    half* d_bias = nullptr;
    int* d_err = nullptr;
    size_t stream_bytes = 0;
};

static int choose_nb(int n_block_rows, int size_hint) {
    const int slabs = std::max(1, (size_hint + kSlab - 1) / kSlab);
    const int target = sm_count() * 9 / 10;
    for (int nb : {24, 16, 12, 8}) {
        const int chunks = (n_block_rows + nb - 1) / nb;
        if ((long)slabs * chunks >= target) return std::min(nb, std::max(n_block_rows, 1));
    }
    return std::min(8, std::max(n_block_rows, 1));
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
    w->K = K; w->N = N; w->ntile = ntile;
    w->nb = nb_override > 0 ? std::min(nb_override, kMaxNB) : choose_nb(NBR, size_hint);
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
    w->stage_b_bytes = (int)((max_block + 1023) / 1024 * 1024);
    const int stage = kXStageBytes + w->stage_b_bytes;
    w->num_stages = std::min(kMaxStages, (kSmemMax - 1024 - (int)sizeof(Shared)) / stage);
    if (w->num_stages < 2) { delete w; return fail(ET_ERR_UNSUPPORTED, "tile weight: weight block exceeds shared memory"); }
    w->num_stages = std::min(w->num_stages, std::max(2, w->k_chunks));
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
    CUtensorMap tm;
    if (!make_tmap_2d_f16(&tm, X, (uint64_t)T, (uint64_t)w->K, (uint64_t)w->K, kSlab, kKC, true))
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
    p.stage_b_bytes = w->stage_b_bytes; p.num_stages = w->num_stages; p.gelu = gelu; p.err = w->d_err;
    p.prof = g_prof;
    const size_t smem = (size_t)w->num_stages * (kXStageBytes + w->stage_b_bytes) + sizeof(Shared) + 1024;
    dim3 grid((T + kSlab - 1) / kSlab, w->n_chunks);
    tile_gemm_kernel<<<grid, kThreads, smem, st>>>(tm, p);
    return cuda_status(cudaGetLastError(), "tile linear launch");
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
    info[0] = w->nb; info[1] = w->n_chunks; info[2] = w->k_chunks; info[3] = w->num_stages;
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
