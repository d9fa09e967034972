// Host-side layer objects: the row-pruned linear and the three encoder-layer variants, plus their
// C-ABI entry points. Replaces encoder/Linear.cu:60-91 (Linear_row), encoder/encoder.h:7-134 and
// encoder/encoder.cu:4-149 (Encoder_base / Encoder_tile / Encoder_prune / Encoder_length) of the reference.
//
// Differences from the reference by design: one stream, no host synchronisation inside run(), no cuBLAS;
// a batch of packed variable-length sequences is a first-class input (run_batch); every failure is a
// status code instead of exit(1).
#include <algorithm>
#include <map>
#include <memory>
#include <mutex>
#include <tuple>
#include <vector>
#include "attention.h"
#include "common.h"
#include "formats.h"
#include "handles.h"
#include "tile_gemm.h"


namespace et {

// ------------------------------------------------------------------------------ row-pruned linear
// Only `row_id_size` output features survive (sorted original indices in row_id); the weight is the
// compact [row_id_size x in_feat] matrix. Output is [tokens x nrow] with nrow = row_id_size rounded up
// to 16 (zero columns beyond row_id_size), the pitch every consumer uses. The contraction runs on the
// tile kernel with every tile kept.
struct RowWeight {
    int in_feat = 0, out_feat = 0, nhead = 0, row_id_size = 0, nrow = 0;
    TileWeight* tw = nullptr;
    int* d_row_id = nullptr;
    int* d_head_ptr = nullptr;
    int* d_inv = nullptr;   // [out_feat]: compact column of an original feature, -1 where it was pruned
    std::vector<int> h_head_ptr;
    ~RowWeight() {
        tile_weight_free(tw);
        cudaFree(d_row_id);
        cudaFree(d_head_ptr);
        cudaFree(d_inv);
    }
};

static int dense_to_tiles(const half* weight, int rows, int K, std::vector<half>& data,
                          std::vector<int>& row_ptr, std::vector<int>& row_offset) {
    const int nrow = (rows + 15) / 16 * 16;
    const int brs = nrow / 16, bcs = K / 16;
    data.assign((size_t)brs * bcs * 256, __float2half(0.f));
    row_ptr.resize(brs + 1);
    row_offset.resize((size_t)brs * bcs);
    for (int r = 0; r < brs; ++r) {
        row_ptr[r] = r * bcs;
        for (int c = 0; c < bcs; ++c) {
            const size_t i = (size_t)r * bcs + c;
            row_offset[i] = c * 16;
            for (int n = 0; n < 16 && 16 * r + n < rows; ++n)
                for (int k = 0; k < 16; ++k)
                    data[i * 256 + n * 16 + k] = weight[(size_t)(16 * r + n) * K + 16 * c + k];
        }
    }
    row_ptr[brs] = brs * bcs;
    return nrow;
}

static int row_weight_create(RowWeight** out, int in_feat, int out_feat, int size, const half* weight,
                             const int* row_id, int row_id_size, const half* bias, int nhead) {
    if (!out) return fail(ET_ERR_INVALID, "row weight: null output");
    *out = nullptr;
    if (in_feat <= 0 || in_feat % 16 || out_feat <= 0 || row_id_size <= 0 || row_id_size > out_feat)
        return fail(ET_ERR_INVALID, "row weight: bad dimensions (in_feat must be a multiple of 16)");
    if (!weight || !row_id) return fail(ET_ERR_INVALID, "row weight: null array");
    if (nhead <= 0 || out_feat % nhead) return fail(ET_ERR_INVALID, "row weight: out_feat not divisible by nhead");
    for (int i = 0; i < row_id_size; ++i)
        if (row_id[i] < 0 || row_id[i] >= out_feat || (i && row_id[i] <= row_id[i - 1]))
            return fail(ET_ERR_INVALID, "row weight: row_id must be strictly ascending inside [0, out_feat)");
    auto w = std::make_unique<RowWeight>();
    w->in_feat = in_feat; w->out_feat = out_feat; w->nhead = nhead; w->row_id_size = row_id_size;
    std::vector<half> data;
    std::vector<int> rp, ro;
    w->nrow = dense_to_tiles(weight, row_id_size, in_feat, data, rp, ro);
    std::vector<half> pbias(w->nrow, __float2half(0.f));
    if (bias) std::copy(bias, bias + row_id_size, pbias.begin());
    int rc = tile_weight_pack(&w->tw, in_feat, w->nrow, size, (long)ro.size(), data.data(), rp.data(),
                              ro.data(), pbias.data(), 0);
    if (rc) return rc;
    build_head_ptr(row_id, row_id_size, nhead, out_feat, w->h_head_ptr);
    if (cudaMalloc(&w->d_row_id, sizeof(int) * row_id_size) != cudaSuccess ||
        cudaMalloc(&w->d_head_ptr, sizeof(int) * (nhead + 1)) != cudaSuccess)
        return fail(ET_ERR_CUDA, "row weight: cudaMalloc failed");
    cudaMemcpy(w->d_row_id, row_id, sizeof(int) * row_id_size, cudaMemcpyHostToDevice);
    cudaMemcpy(w->d_head_ptr, w->h_head_ptr.data(), sizeof(int) * (nhead + 1), cudaMemcpyHostToDevice);
    {
        std::vector<int> inv((size_t)(out_feat + 7) / 8 * 8, -1);
        for (int i = 0; i < row_id_size; ++i) inv[row_id[i]] = i;
        if (cudaMalloc(&w->d_inv, sizeof(int) * inv.size()) != cudaSuccess) return fail(ET_ERR_CUDA, "row weight: cudaMalloc failed");
        cudaMemcpy(w->d_inv, inv.data(), sizeof(int) * inv.size(), cudaMemcpyHostToDevice);
    }
    *out = w.release();
    return ET_OK;
}

namespace {
std::mutex g_row_mu;
std::map<std::tuple<const void*, int, int>, TileWeight*> g_row_cache;
}  // namespace

int row_spmm_raw(half* out, const half* in, const half* weight, const half* bias, int M, int N, int K, cudaStream_t st) {
    TileWeight* tw = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_row_mu);
        auto key = std::make_tuple((const void*)weight, N, K);
        auto it = g_row_cache.find(key);
        if (it == g_row_cache.end()) {
            std::vector<half> hw((size_t)N * K);
            if (cudaMemcpy(hw.data(), weight, hw.size() * sizeof(half), cudaMemcpyDeviceToHost) != cudaSuccess)
                return fail(ET_ERR_CUDA, "row spmm: cannot read the weight");
            std::vector<half> data;
            std::vector<int> rp, ro;
            dense_to_tiles(hw.data(), N, K, data, rp, ro);
            int rc = tile_weight_pack(&tw, K, N, M, (long)ro.size(), data.data(), rp.data(), ro.data(), nullptr, 0);
            if (rc) return rc;
            g_row_cache[key] = tw;
        } else {
            tw = it->second;
        }
    }
    return tile_linear_run(tw, out, in, M, 0, st, bias);
}

void row_spmm_cache_clear() {
    std::lock_guard<std::mutex> lk(g_row_mu);
    for (auto& kv : g_row_cache) tile_weight_free(kv.second);
    g_row_cache.clear();
}

// ------------------------------------------------------------------------------ encoder layer
enum EncoderKind { kTile = 0, kPrune = 1, kLength = 2, kPruneQKV = 3 };

// The legacy default stream cannot be captured, so a layer launched there could not be replayed as a CUDA graph
// (and its seven launches would cost the host three times as much). Calls on the legacy stream therefore run on a
// stream of the object, ordered behind the caller's stream by one event and ahead of it by another.
struct StreamBridge {
    cudaStream_t own = nullptr;
    cudaEvent_t in = nullptr, out = nullptr;
    ~StreamBridge() {
        if (in) cudaEventDestroy(in);
        if (out) cudaEventDestroy(out);
        if (own) cudaStreamDestroy(own);
    }
    static bool is_legacy(cudaStream_t st) { return st == nullptr || st == cudaStreamLegacy; }
    // Returns the stream to run on, or nullptr if the bridge could not be set up (the caller then stays on `st`).
    cudaStream_t begin(cudaStream_t st) {
        if (!own) {
            if (cudaStreamCreateWithFlags(&own, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&in, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&out, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                return nullptr;
            }
        }
        if (cudaEventRecord(in, st) != cudaSuccess || cudaStreamWaitEvent(own, in, 0) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return own;
    }
    void end(cudaStream_t st) {
        if (cudaEventRecord(out, own) != cudaSuccess || cudaStreamWaitEvent(st, out, 0) != cudaSuccess) cudaGetLastError();
    }
};

struct Encoder {
    int kind = kTile, d_model = 0, seq_len = 0, nheads = 0, d_ff = 0;
    half* buffer = nullptr;  // caller-owned scratch for run(): buffer_num * seq_len * d_model halfs (+ scores)
    TileWeight* lin[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // q k v o mlp1 mlp2
    TileWeight* qkv = nullptr;   // Q|K|V as one weight: one launch, one staging of the activations per CTA
    int qkv_cols[3] = {0, 0, 0}; // output columns of the three parts inside the fused result
    bool expand_pruned = false;  // row-pruned operands are expanded to their original positions (zeros where pruned)
                                 // and attention runs on the tensor-core kernel
    RowWeight* rq = nullptr; RowWeight* rk = nullptr; RowWeight* rv = nullptr;
    half* d_ln[4] = {nullptr, nullptr, nullptr, nullptr};  // gamma1 beta1 gamma2 beta2
    std::vector<half> h_ln[4];                             // the same on the host (folded into weights by the layer stack)
    half* d_mask = nullptr;                                // [seq_len x seq_len] additive, may be null
    int* d_lens = nullptr; int lens_cap = 0;               // cu_seqlens (batch+1) then valid_lens (batch)
    bool materialize_scores = false;
    // Replay cache: one instantiated CUDA graph per distinct call (buffers, lengths). A layer is 7 short
    // launches; replaying them as one graph removes the launch gaps between them.
    struct Replay {
        std::vector<int64_t> key;
        int seen = 0;
        cudaGraphExec_t exec = nullptr;
    };
    std::vector<Replay> replays;
    bool use_graphs = true;
    StreamBridge bridge;
    void drop_replays() {
        for (auto& r : replays)
            if (r.exec) cudaGraphExecDestroy(r.exec);
        replays.clear();
    }
    ~Encoder() {
        drop_replays();
        for (auto* t : lin) tile_weight_free(t);
        tile_weight_free(qkv);
        delete rq; delete rk; delete rv;
        for (auto* p : d_ln) cudaFree(p);
        cudaFree(d_mask);
        cudaFree(d_lens);
    }
};

// The device array of sequence offsets and key counts grows geometrically. A recorded graph holds the array's
// address as a kernel argument, so every graph recorded with the old array is dropped before it is freed
// (`drop` does that); the caller re-records on its next calls.
template <typename Drop>
static int grow_lens(int** d_lens, int* cap, int need, Drop&& drop) {
    if (*cap >= need) return ET_OK;
    drop();
    int ncap = std::max(need, std::max(64, 2 * *cap));
    int* fresh = nullptr;
    if (cudaMalloc(&fresh, sizeof(int) * (size_t)ncap) != cudaSuccess) return fail(ET_ERR_CUDA, "lengths: cudaMalloc failed");
    cudaFree(*d_lens);   // synchronises with work still reading the old array
    *d_lens = fresh;
    *cap = ncap;
    return ET_OK;
}

static int upload_half(half** dst, const half* src_host, size_t n) {
    if (cudaMalloc(dst, n * sizeof(half)) != cudaSuccess) return fail(ET_ERR_CUDA, "encoder: cudaMalloc failed");
    return cuda_status(cudaMemcpy(*dst, src_host, n * sizeof(half), cudaMemcpyHostToDevice), "encoder: upload");
}

static int encoder_common(Encoder* e, int d_model, int seq_len, int nheads, half* buffer,
                          const half* g1, const half* b1, const half* g2, const half* b2, const half* mask) {
    if (d_model <= 0 || seq_len <= 0 || nheads <= 0 || d_model % nheads) return fail(ET_ERR_INVALID, "encoder: bad dimensions");
    if (!g1 || !b1 || !g2 || !b2) return fail(ET_ERR_INVALID, "encoder: null LayerNorm parameter");
    {
        // nothing is left to set up when the first attention launch comes (it may sit inside a caller's capture)
        const int rc = attention_prepare_device();
        if (rc) return rc;
    }
    e->d_model = d_model; e->seq_len = seq_len; e->nheads = nheads; e->buffer = buffer;
    const half* src[4] = {g1, b1, g2, b2};
    for (int i = 0; i < 4; ++i) {
        int rc = upload_half(&e->d_ln[i], src[i], d_model);
        if (rc) return rc;
        e->h_ln[i].assign(src[i], src[i] + d_model);
    }
    if (mask) return upload_half(&e->d_mask, mask, (size_t)seq_len * seq_len);
    return ET_OK;
}

// One layer over `T` packed tokens (op order of encoder/encoder.cu:20-45). scratch holds 5*T*d_model halfs:
// [0] Q then the attention-output projection / first LayerNorm result, [1] K, [2] V, [3] attention output,
// [1..4] the T x d_ff hidden activations; scores (materialised variant) follow at 5*T*d_model.
static int encoder_forward(Encoder* e, half* out, const half* in, half* scratch, int T, const int* cu_seqlens,
                           const int* valid_lens, int batch, int uniform_len, cudaStream_t st, int max_len = 0) {
    const size_t td = (size_t)T * e->d_model;
    half* b0 = scratch; half* b1 = scratch + td; half* b2 = scratch + 2 * td; half* b3 = scratch + 3 * td;
    int rc;
    int q_pitch = e->d_model, v_pitch = e->d_model;
    const int *qk_hp = nullptr, *v_hp = nullptr, *v_id = nullptr;
    if (e->qkv && e->expand_pruned) {
        // Row-pruned operands. One launch writes the compact Q | K | V side by side; one bandwidth-bound pass puts
        // the row-pruned ones back at their original feature positions with zeros where a feature was pruned; the
        // tensor-core attention kernel then runs on dense heads of 64: a zero column adds nothing to Q K^T, and a
        // zero column of V gives a zero column of the result, which is the scatter with zero fill that the pruned
        // attention means (kernels/attention.cu:242-248).
        const int P = e->qkv_cols[0] + e->qkv_cols[1] + e->qkv_cols[2];
        const int d = e->d_model;
        half* b4 = scratch + 4 * td;
        if (e->kind == kPruneQKV) {
            // compact result in buffers 3-4 (P <= 2 d_model), expanded Q | K | V over buffers 0-2
            half* comp = b3;
            if ((rc = tile_linear_run(e->qkv, comp, in, T, 0, st))) return rc;
            const half* src[3] = {comp, comp + e->qkv_cols[0], comp + e->qkv_cols[0] + e->qkv_cols[1]};
            const int sp[3] = {P, P, P}, dp[3] = {3 * d, 3 * d, 3 * d};
            half* dst[3] = {b0, b0 + d, b0 + 2 * d};
            const int* inv[3] = {e->rq->d_inv, e->rk->d_inv, e->rv->d_inv};
            if ((rc = expand_rows_launch(3, src, sp, dst, dp, inv, d, T, st))) return rc;
            q_pitch = v_pitch = 3 * d;
            b1 = b0 + d;
            b2 = b0 + 2 * d;
        } else {
            // Q and K are dense already (inside the fused result); only V is expanded, into buffer 4
            if ((rc = tile_linear_run(e->qkv, b0, in, T, 0, st))) return rc;
            const half* src[1] = {b0 + e->qkv_cols[0] + e->qkv_cols[1]};
            const int sp[1] = {P}, dp[1] = {d};
            half* dst[1] = {b4};
            const int* inv[1] = {e->rv->d_inv};
            if ((rc = expand_rows_launch(1, src, sp, dst, dp, inv, d, T, st))) return rc;
            q_pitch = P;
            v_pitch = d;
            b1 = b0 + e->qkv_cols[0];
            b2 = b4;
        }
    } else if (e->qkv) {
        // fused: one launch writes Q | K | V side by side, [T x (q + k + v columns)] over the first three scratch
        // buffers (row-pruned parts are compact, so the three widths may differ)
        if ((rc = tile_linear_run(e->qkv, b0, in, T, 0, st))) return rc;
        q_pitch = v_pitch = e->qkv_cols[0] + e->qkv_cols[1] + e->qkv_cols[2];
        b1 = b0 + e->qkv_cols[0];
        b2 = b1 + e->qkv_cols[1];
        if (e->kind == kPruneQKV) qk_hp = e->rq->d_head_ptr;
        if (e->kind == kPrune || e->kind == kPruneQKV) { v_hp = e->rv->d_head_ptr; v_id = e->rv->d_row_id; }
    } else if (e->kind == kPruneQKV) {
        if ((rc = tile_linear_run(e->rq->tw, b0, in, T, 0, st))) return rc;
        if ((rc = tile_linear_run(e->rk->tw, b1, in, T, 0, st))) return rc;
        q_pitch = e->rq->nrow; qk_hp = e->rq->d_head_ptr;
    } else {
        if ((rc = tile_linear_run(e->lin[0], b0, in, T, 0, st))) return rc;
        if ((rc = tile_linear_run(e->lin[1], b1, in, T, 0, st))) return rc;
    }
    if (e->qkv) {
    } else if (e->kind == kPrune || e->kind == kPruneQKV) {
        if ((rc = tile_linear_run(e->rv->tw, b2, in, T, 0, st))) return rc;
        v_pitch = e->rv->nrow; v_hp = e->rv->d_head_ptr; v_id = e->rv->d_row_id;
    } else {
        if ((rc = tile_linear_run(e->lin[2], b2, in, T, 0, st))) return rc;
    }
    const half* scores = nullptr;
    if (e->kind == kLength && e->materialize_scores && !cu_seqlens) {
        half* sbuf = scratch + 5 * td;
        if ((rc = qk_scores_launch(sbuf, b0, b1, batch, uniform_len, e->d_model, e->nheads, st, q_pitch))) return rc;
        scores = sbuf;
    }
    if ((rc = attention_launch(b3, b0, b1, b2, scores, q_pitch, v_pitch, qk_hp, v_id, v_hp, e->d_mask, e->seq_len,
                               cu_seqlens, valid_lens, batch, uniform_len, T, e->d_model, e->nheads, st, max_len)))
        return rc;
    b1 = scratch + td;
    if ((rc = tile_linear_run(e->lin[3], b0, b3, T, 0, st))) return rc;
    if ((rc = et_skip_layernorm(b0, in, e->d_ln[0], e->d_ln[1], T, e->d_model, st))) return rc;
    if ((rc = tile_linear_run(e->lin[4], b1, b0, T, 1, st))) return rc;
    if ((rc = tile_linear_run(e->lin[5], out, b1, T, 0, st))) return rc;
    return et_skip_layernorm(out, b0, e->d_ln[2], e->d_ln[3], T, e->d_model, st);
}


// ------------------------------------------------------------------------------ stack of layers
// N encoder layers run back to back on packed tokens: the caller's side of the reference's one-layer objects
// (test/tile_test.cu:36-41 calls run() once for one layer). The model owns its scratch (grown on demand, kept
// between calls), uploads the lengths once per call, and replays all N x 7 launches as one CUDA graph.
struct Model {
    std::vector<Encoder*> layers;
    half* scratch = nullptr; size_t scratch_halfs = 0;
    int* d_lens = nullptr; int lens_cap = 0;
    struct Replay {
        std::vector<int64_t> key;
        int seen = 0;
        cudaGraphExec_t exec = nullptr;
    };
    std::vector<Replay> replays;
    bool use_graphs = true;
    StreamBridge bridge;
    // LayerNorm folded into the linears (tile and length layers): per layer the FFN1 weight folded with the layer's
    // first LayerNorm, the fused Q|K|V weight folded with the PREVIOUS layer's second LayerNorm, fp32 copies of
    // the four LayerNorm vectors; per row the partial sums that the output projection and FFN2 leave behind.
    struct Fused {
        TileWeight* ffn1 = nullptr;
        TileWeight* qkv = nullptr;
        float* lnf[4] = {nullptr, nullptr, nullptr, nullptr};
        int np1 = 0, np2 = 0;   // partial-sum slots per row of the output projection / of FFN2
    };
    std::vector<Fused> fused;
    bool fuse_ln = false;
    float* stats1 = nullptr; float* stats2 = nullptr; size_t stats_floats = 0;
    void drop_replays() {
        for (auto& r : replays)
            if (r.exec) cudaGraphExecDestroy(r.exec);
        replays.clear();
    }
    void drop_fused() {
        for (auto& f : fused) {
            tile_weight_free(f.ffn1);
            tile_weight_free(f.qkv);
            for (float* p : f.lnf) cudaFree(p);
        }
        fused.clear();
        fuse_ln = false;
    }
    ~Model() {
        drop_replays();
        drop_fused();
        for (auto* e : layers) delete e;
        cudaFree(scratch);
        cudaFree(d_lens);
        cudaFree(stats1);
        cudaFree(stats2);
    }
};

int layernorm_launch(half* x, const half* s, const half* g, const half* b, int num, int size, cudaStream_t st);

// Builds the folded weights. Returns ET_OK with fuse_ln left false when the stack is not eligible (a row-pruned
// layer, or a layer without the fused Q|K|V weight): such stacks run layer by layer with separate LayerNorms.
static int model_prepare_fusion(Model* m) {
    m->drop_fused();
    for (const Encoder* e : m->layers)
        if ((e->kind != kTile && e->kind != kLength) || !e->qkv || (e->d_model & 7)) return ET_OK;
    m->fused.resize(m->layers.size());
    for (size_t l = 0; l < m->layers.size(); ++l) {
        Encoder* e = m->layers[l];
        Model::Fused& f = m->fused[l];
        int rc = tile_weight_fold(&f.ffn1, e->lin[4], e->h_ln[0].data(), e->h_ln[1].data());
        if (rc == ET_OK && l > 0) {
            const Encoder* pe = m->layers[l - 1];
            rc = tile_weight_fold(&f.qkv, e->qkv, pe->h_ln[2].data(), pe->h_ln[3].data());
        }
        if (rc) { m->drop_fused(); return rc; }
        for (int i = 0; i < 4; ++i) {
            std::vector<float> v(e->d_model);
            for (int k = 0; k < e->d_model; ++k) v[k] = __half2float(e->h_ln[i][k]);
            if (cudaMalloc(&f.lnf[i], v.size() * sizeof(float)) != cudaSuccess) { m->drop_fused(); return fail(ET_ERR_CUDA, "model: cudaMalloc failed"); }
            cudaMemcpy(f.lnf[i], v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice);
        }
        f.np1 = tile_weight_stat_slots(e->lin[3]);
        f.np2 = tile_weight_stat_slots(e->lin[5]);
    }
    m->fuse_ln = true;
    return ET_OK;
}

// The stack with its LayerNorms folded into the linears. Per layer: fused Q|K|V (normalising its input in the
// epilogue from layer 1 on), attention, output projection + residual -> y1 and its row sums, FFN1 (normalises y1 in
// the epilogue, GELU), FFN2 + LayerNorm(y1) as residual -> y2 and its row sums into `out`; the next layer reads
// `out` un-normalised. One plain LayerNorm of `out` ends the stack. 5 launches per layer instead of 7.
static int model_forward_fused(Model* m, half* out, const half* in, int T, const int* cu, const int* vl, int batch,
                               int uniform_len, cudaStream_t st, int max_len) {
    half* scratch = m->scratch;
    const half* yprev = in;
    int rc;
    for (size_t l = 0; l < m->layers.size(); ++l) {
        Encoder* e = m->layers[l];
        const Model::Fused& f = m->fused[l];
        const int d = e->d_model;
        const size_t td = (size_t)T * d;
        half* b0 = scratch; half* b3 = scratch + 3 * td;
        half* b1 = scratch + td;
        if (l == 0) {
            if ((rc = tile_linear_run(e->qkv, b0, in, T, 0, st))) return rc;
        } else {
            GemmFusion fz;
            fz.mode = 1; fz.stats_in = m->stats2; fz.np_in = m->fused[l - 1].np2;
            if ((rc = tile_linear_run(f.qkv, b0, yprev, T, 0, st, nullptr, &fz))) return rc;
        }
        const half* scores = nullptr;
        if (e->kind == kLength && e->materialize_scores && !cu) {
            half* sbuf = scratch + 5 * td;
            if ((rc = qk_scores_launch(sbuf, b0, b0 + d, batch, uniform_len, d, e->nheads, st, 3 * d))) return rc;
            scores = sbuf;
        }
        if ((rc = attention_launch(b3, b0, b0 + d, b0 + 2 * d, scores, 3 * d, 3 * d, nullptr, nullptr, nullptr, e->d_mask,
                                   e->seq_len, cu, vl, batch, uniform_len, T, d, e->nheads, st, max_len)))
            return rc;
        {   // y1 = Z Wo^T + bo + residual
            GemmFusion fz;
            fz.resid = yprev; fz.stats_out = m->stats1; fz.np_out = f.np1;
            if (l == 0) {
                fz.mode = 2;
            } else {
                const Model::Fused& pf = m->fused[l - 1];
                fz.mode = 3; fz.stats_src = m->stats2; fz.np_src = pf.np2; fz.gamma_s = pf.lnf[2]; fz.beta_s = pf.lnf[3];
            }
            if ((rc = tile_linear_run(e->lin[3], b0, b3, T, 0, st, nullptr, &fz))) return rc;
        }
        {   // F = gelu(LN1(y1) W1^T + b1)
            GemmFusion fz;
            fz.mode = 1; fz.stats_in = m->stats1; fz.np_in = f.np1;
            if ((rc = tile_linear_run(f.ffn1, b1, b0, T, 1, st, nullptr, &fz))) return rc;
        }
        {   // y2 = F W2^T + b2 + LN1(y1)
            GemmFusion fz;
            fz.mode = 3; fz.resid = b0; fz.stats_src = m->stats1; fz.np_src = f.np1; fz.gamma_s = f.lnf[0]; fz.beta_s = f.lnf[1];
            fz.stats_out = m->stats2; fz.np_out = f.np2;
            if ((rc = tile_linear_run(e->lin[5], out, b1, T, 0, st, nullptr, &fz))) return rc;
        }
        yprev = out;
    }
    const Encoder* last = m->layers.back();
    return layernorm_launch(out, nullptr, last->d_ln[2], last->d_ln[3], T, last->d_model, st);
}

static size_t model_scratch_halfs(const Model* m, int total_tokens, int batch, int max_len) {
    size_t need = 0;
    for (const Encoder* e : m->layers) {
        size_t n = (size_t)5 * e->d_model * total_tokens;
        if (e->kind == kLength && e->materialize_scores) n += (size_t)batch * e->nheads * max_len * max_len;
        need = std::max(need, n);
    }
    return need;
}

static int model_forward(Model* m, half* out, const half* in, int T, const int* cu, const int* vl, int batch,
                         int uniform_len, cudaStream_t st, int max_len) {
    if (m->fuse_ln) return model_forward_fused(m, out, in, T, cu, vl, batch, uniform_len, st, max_len);
    const half* x = in;
    for (Encoder* e : m->layers) {
        // a layer may write over its own input (the input is consumed before the last two launches write `out`)
        const int rc = encoder_forward(e, out, x, m->scratch, T, cu, vl, batch, uniform_len, st, max_len);
        if (rc) return rc;
        x = out;
    }
    return ET_OK;
}

}  // namespace et

using et::Encoder;
using et::RowWeight;

struct et_row_weight {
    RowWeight* w;
};
struct et_encoder {
    Encoder* e;
};

extern "C" {

int et_row_weight_create(et_row_weight** out, int in_feat, int out_feat, int size, const void* weight_host,
                         const int* row_id_host, int row_id_size, const void* bias_host, int nhead) {
    ET_REQUIRE(out, "et_row_weight_create: null output");
    *out = nullptr;
    RowWeight* w = nullptr;
    int rc = et::row_weight_create(&w, in_feat, out_feat, size, static_cast<const half*>(weight_host), row_id_host,
                                   row_id_size, static_cast<const half*>(bias_host), nhead);
    if (rc) { delete w; return rc; }
    *out = new et_row_weight{w};
    return ET_OK;
}
int et_row_weight_destroy(et_row_weight* w) {
    if (w) { delete w->w; delete w; }
    return ET_OK;
}
int et_row_linear(const et_row_weight* w, void* out, const void* in, int tokens, void* stream) {
    ET_REQUIRE(w, "et_row_linear: null weight");
    return et::tile_linear_run(w->w->tw, static_cast<half*>(out), static_cast<const half*>(in), tokens, 0,
                               static_cast<cudaStream_t>(stream));
}
// Launcher-level form with a DEVICE-resident dense compact weight [N x K] (N a multiple of 16 as the
// reference pads it). The packed form is built on first use (device-to-host copy, synchronous) and cached
// by weight address; et_tile_spmm_cache_clear() drops these entries too.
int et_row_spmm_bias(void* out, const void* in, const void* weight, const void* bias, int M, int N, int K,
                     void* stream) {
    ET_REQUIRE(out && in && weight && bias, "et_row_spmm_bias: null pointer");
    ET_REQUIRE(N > 0 && K > 0 && N % 16 == 0 && K % 16 == 0, "et_row_spmm_bias: N and K must be positive multiples of 16");
    return et::row_spmm_raw(static_cast<half*>(out), static_cast<const half*>(in), static_cast<const half*>(weight),
                            static_cast<const half*>(bias), M, N, K, static_cast<cudaStream_t>(stream));
}
int et_row_weight_meta(const et_row_weight* w, int* nrow, int* row_id_size, const int** row_id_dev,
                       const int** head_ptr_dev, int* head_ptr_host) {
    ET_REQUIRE(w, "et_row_weight_meta: null weight");
    if (nrow) *nrow = w->w->nrow;
    if (row_id_size) *row_id_size = w->w->row_id_size;
    if (row_id_dev) *row_id_dev = w->w->d_row_id;
    if (head_ptr_dev) *head_ptr_dev = w->w->d_head_ptr;
    if (head_ptr_host) std::copy(w->w->h_head_ptr.begin(), w->w->h_head_ptr.end(), head_ptr_host);
    return ET_OK;
}

int et_attention_otf(void* out, const void* Q, const void* K, const void* V, const void* mask, int seq_len,
                     int d_model, int nhead, void* stream) {
    ET_REQUIRE(seq_len >= 0, "et_attention_otf: negative seq_len");
    return et::attention_launch(static_cast<half*>(out), static_cast<const half*>(Q), static_cast<const half*>(K),
                                static_cast<const half*>(V), nullptr, d_model, d_model, nullptr, nullptr, nullptr,
                                static_cast<const half*>(mask), seq_len, nullptr, nullptr, 1, seq_len, seq_len,
                                d_model, nhead, static_cast<cudaStream_t>(stream));
}
int et_attention_prune(void* out, const void* Q, const void* K, const void* V, const int* v_col_id,
                       const int* v_head_ptr, int nnz_col_v, const void* mask, int seq_len, int d_model,
                       int nhead, void* stream) {
    ET_REQUIRE(seq_len >= 0 && nnz_col_v > 0, "et_attention_prune: bad dimensions");
    ET_REQUIRE(v_col_id && v_head_ptr, "et_attention_prune: null index array");
    return et::attention_launch(static_cast<half*>(out), static_cast<const half*>(Q), static_cast<const half*>(K),
                                static_cast<const half*>(V), nullptr, d_model, nnz_col_v, nullptr, v_col_id,
                                v_head_ptr, static_cast<const half*>(mask), seq_len, nullptr, nullptr, 1, seq_len,
                                seq_len, d_model, nhead, static_cast<cudaStream_t>(stream));
}
int et_qk_scores(void* QK, const void* Q, const void* K, int seq_len, int d_model, int nhead, void* stream) {
    return et::qk_scores_launch(static_cast<half*>(QK), static_cast<const half*>(Q), static_cast<const half*>(K), 1,
                                seq_len, d_model, nhead, static_cast<cudaStream_t>(stream));
}
int et_attention_sharedqk(void* out, const void* QK, const void* V, const void* mask, int seq_len, int d_model,
                          int nhead, void* stream) {
    ET_REQUIRE(QK, "et_attention_sharedqk: null scores");
    return et::attention_launch(static_cast<half*>(out), nullptr, nullptr, static_cast<const half*>(V),
                                static_cast<const half*>(QK), d_model, d_model, nullptr, nullptr, nullptr,
                                static_cast<const half*>(mask), seq_len, nullptr, nullptr, 1, seq_len, seq_len,
                                d_model, nhead, static_cast<cudaStream_t>(stream));
}
int et_attention_static_scores(void* out, const void* Q, const void* K, const void* V, const void* mask,
                               int seq_len, int d_model, int nhead, void* stream) {
    ET_REQUIRE(out && Q && K && V, "et_attention_static_scores: null pointer");
    return et::attention_static_scores(static_cast<half*>(out), static_cast<const half*>(Q),
                                       static_cast<const half*>(K), static_cast<const half*>(V),
                                       static_cast<const half*>(mask), seq_len, d_model, nhead,
                                       static_cast<cudaStream_t>(stream));
}
int et_attention_batch(void* out, const void* Q, const void* K, const void* V, int qk_pitch, int v_pitch,
                       const int* qk_head_ptr, const int* v_col_id, const int* v_head_ptr, const void* mask,
                       int mask_ld, const int* cu_seqlens, const int* valid_lens, int batch, int uniform_len,
                       int max_seq_len, int total_tokens, int d_model, int nhead, void* stream) {
    return et::attention_launch(static_cast<half*>(out), static_cast<const half*>(Q), static_cast<const half*>(K),
                                static_cast<const half*>(V), nullptr, qk_pitch, v_pitch, qk_head_ptr, v_col_id,
                                v_head_ptr, static_cast<const half*>(mask), mask_ld, cu_seqlens, valid_lens, batch,
                                uniform_len, total_tokens, d_model, nhead, static_cast<cudaStream_t>(stream),
                                max_seq_len);
}

// ------------------------------------------------------------------------------ encoders
static int take_tiles(Encoder* e, et_tile_weight** t, int first, int count, int d_model) {
    for (int i = 0; i < count; ++i)
        if (!t[i] || !t[i]->w) return et::fail(ET_ERR_INVALID, "encoder: null linear");
    for (int i = 0; i < count; ++i) {
        e->lin[first + i] = t[i]->w;   // ownership moves into the encoder, as the reference's rvalue ctor
        t[i]->w = nullptr;
    }
    (void)d_model;
    return ET_OK;
}

static int finish_create(et_encoder** out, std::unique_ptr<Encoder>& e) {
    *out = new et_encoder{e.release()};
    return ET_OK;
}

int et_encoder_tile_create(et_encoder** out, int kind, int d_model, int seq_len, int nheads, void* buffer,
                           et_tile_weight* q, et_tile_weight* k, et_tile_weight* v, et_tile_weight* o,
                           et_tile_weight* mlp1, et_tile_weight* mlp2, const void* ln_gamma_1,
                           const void* ln_beta_1, const void* ln_gamma_2, const void* ln_beta_2,
                           const void* mask_host) {
    ET_REQUIRE(out, "et_encoder_tile_create: null output");
    *out = nullptr;
    ET_REQUIRE(kind == et::kTile || kind == et::kLength, "et_encoder_tile_create: kind must be 0 (tile) or 2 (length)");
    auto e = std::make_unique<Encoder>();
    e->kind = kind;
    int rc = et::encoder_common(e.get(), d_model, seq_len, nheads, static_cast<half*>(buffer),
                                static_cast<const half*>(ln_gamma_1), static_cast<const half*>(ln_beta_1),
                                static_cast<const half*>(ln_gamma_2), static_cast<const half*>(ln_beta_2),
                                static_cast<const half*>(mask_host));
    if (rc) return rc;
    et_tile_weight* t[6] = {q, k, v, o, mlp1, mlp2};
    if ((rc = take_tiles(e.get(), t, 0, 6, d_model))) return rc;
    if (et::tile_weight_out_feat(e->lin[0]) == d_model && et::tile_weight_out_feat(e->lin[1]) == d_model &&
        et::tile_weight_out_feat(e->lin[2]) == d_model) {
        const et::TileWeight* parts[3] = {e->lin[0], e->lin[1], e->lin[2]};
        if ((rc = et::tile_weight_concat(&e->qkv, parts, 3, 0))) return rc;
        for (int i = 0; i < 3; ++i) e->qkv_cols[i] = d_model;
    }
    return finish_create(out, e);
}

int et_encoder_prune_create(et_encoder** out, int d_model, int seq_len, int nheads, void* buffer,
                            et_tile_weight* q, et_tile_weight* k, et_row_weight* v, et_tile_weight* o,
                            et_tile_weight* mlp1, et_tile_weight* mlp2, const void* ln_gamma_1,
                            const void* ln_beta_1, const void* ln_gamma_2, const void* ln_beta_2,
                            const void* mask_host) {
    ET_REQUIRE(out, "et_encoder_prune_create: null output");
    *out = nullptr;
    ET_REQUIRE(v && v->w, "et_encoder_prune_create: null V linear");
    auto e = std::make_unique<Encoder>();
    e->kind = et::kPrune;
    int rc = et::encoder_common(e.get(), d_model, seq_len, nheads, static_cast<half*>(buffer),
                                static_cast<const half*>(ln_gamma_1), static_cast<const half*>(ln_beta_1),
                                static_cast<const half*>(ln_gamma_2), static_cast<const half*>(ln_beta_2),
                                static_cast<const half*>(mask_host));
    if (rc) return rc;
    et_tile_weight* t01[2] = {q, k};
    et_tile_weight* t35[3] = {o, mlp1, mlp2};
    if ((rc = take_tiles(e.get(), t01, 0, 2, d_model))) return rc;
    if ((rc = take_tiles(e.get(), t35, 3, 3, d_model))) return rc;
    e->rv = v->w; v->w = nullptr;
    if (et::tile_weight_out_feat(e->lin[0]) == d_model && et::tile_weight_out_feat(e->lin[1]) == d_model &&
        e->rv->in_feat == d_model) {
        // Q | K | compact V in one launch
        const et::TileWeight* parts[3] = {e->lin[0], e->lin[1], e->rv->tw};
        if ((rc = et::tile_weight_concat(&e->qkv, parts, 3, 0))) return rc;
        e->qkv_cols[0] = e->qkv_cols[1] = d_model;
        e->qkv_cols[2] = e->rv->nrow;
        e->expand_pruned = d_model / nheads == 64 && e->rv->out_feat == d_model;   // the tensor-core kernel's head width
    }
    return finish_create(out, e);
}

int et_encoder_prune_qkv_create(et_encoder** out, int d_model, int seq_len, int nheads, void* buffer,
                                et_row_weight* q, et_row_weight* k, et_row_weight* v, et_tile_weight* o,
                                et_tile_weight* mlp1, et_tile_weight* mlp2, const void* ln_gamma_1,
                                const void* ln_beta_1, const void* ln_gamma_2, const void* ln_beta_2,
                                const void* mask_host) {
    ET_REQUIRE(out, "et_encoder_prune_qkv_create: null output");
    *out = nullptr;
    ET_REQUIRE(q && q->w && k && k->w && v && v->w, "et_encoder_prune_qkv_create: null linear");
    ET_REQUIRE(q->w->row_id_size == k->w->row_id_size && q->w->h_head_ptr == k->w->h_head_ptr,
               "et_encoder_prune_qkv_create: Q and K must retain the same dimensions per head");
    auto e = std::make_unique<Encoder>();
    e->kind = et::kPruneQKV;
    int rc = et::encoder_common(e.get(), d_model, seq_len, nheads, static_cast<half*>(buffer),
                                static_cast<const half*>(ln_gamma_1), static_cast<const half*>(ln_beta_1),
                                static_cast<const half*>(ln_gamma_2), static_cast<const half*>(ln_beta_2),
                                static_cast<const half*>(mask_host));
    if (rc) return rc;
    et_tile_weight* t35[3] = {o, mlp1, mlp2};
    if ((rc = take_tiles(e.get(), t35, 3, 3, d_model))) return rc;
    e->rq = q->w; q->w = nullptr;
    e->rk = k->w; k->w = nullptr;
    e->rv = v->w; v->w = nullptr;
    if (e->rq->in_feat == d_model && e->rk->in_feat == d_model && e->rv->in_feat == d_model &&
        e->rq->nrow + e->rk->nrow + e->rv->nrow <= 3 * d_model) {
        // compact Q | K | V in one launch
        const et::TileWeight* parts[3] = {e->rq->tw, e->rk->tw, e->rv->tw};
        if ((rc = et::tile_weight_concat(&e->qkv, parts, 3, 0))) return rc;
        e->qkv_cols[0] = e->rq->nrow; e->qkv_cols[1] = e->rk->nrow; e->qkv_cols[2] = e->rv->nrow;
        e->expand_pruned = d_model / nheads == 64 && e->rq->out_feat == d_model && e->rk->out_feat == d_model &&
                           e->rv->out_feat == d_model && e->rq->nrow + e->rk->nrow + e->rv->nrow <= 2 * d_model;
    }
    return finish_create(out, e);
}

int et_encoder_destroy(et_encoder* enc) {
    if (enc) { delete enc->e; delete enc; }
    return ET_OK;
}

int et_encoder_set_materialize_scores(et_encoder* enc, int on) {
    ET_REQUIRE(enc && enc->e, "et_encoder_set_materialize_scores: null encoder");
    ET_REQUIRE(enc->e->kind == et::kLength, "et_encoder_set_materialize_scores: only the length encoder has that path");
    enc->e->materialize_scores = on != 0;
    return ET_OK;
}

size_t et_encoder_buffer_size(int kind, int d_model, int seq_len, int nheads) {
    size_t n = (size_t)5 * d_model * seq_len;
    if (kind == et::kLength) n += (size_t)nheads * seq_len * seq_len;
    return n * sizeof(half);
}

size_t et_encoder_batch_buffer_size(int kind, int d_model, int total_tokens, int batch, int max_len, int nheads) {
    size_t n = (size_t)5 * d_model * total_tokens;
    if (kind == et::kLength) n += (size_t)batch * nheads * max_len * max_len;
    return n * sizeof(half);
}

int et_encoder_run(et_encoder* enc, void* out, const void* in, void* stream) {
    ET_REQUIRE(enc && enc->e && out && in, "et_encoder_run: null pointer");
    Encoder* e = enc->e;
    ET_REQUIRE(e->buffer, "et_encoder_run: the encoder was created without a scratch buffer");
    return et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in), e->buffer, e->seq_len,
                               nullptr, nullptr, 1, e->seq_len, static_cast<cudaStream_t>(stream));
}

int et_encoder_run_batch(et_encoder* enc, void* out, const void* in, const int* seq_lens_host,
                         const int* valid_lens_host, int batch, void* scratch, size_t scratch_bytes, void* stream) {
    ET_REQUIRE(enc && enc->e && out && in && scratch, "et_encoder_run_batch: null pointer");
    ET_REQUIRE(batch >= 0, "et_encoder_run_batch: negative batch");
    Encoder* e = enc->e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (batch == 0) return ET_OK;
    ET_REQUIRE(seq_lens_host, "et_encoder_run_batch: null seq_lens");
    if (e->use_graphs && et::StreamBridge::is_legacy(st)) {
        // the legacy default stream cannot be captured: run on the encoder's own stream, ordered by events
        cudaStream_t own = e->bridge.begin(st);
        if (own) {
            const int rc = et_encoder_run_batch(enc, out, in, seq_lens_host, valid_lens_host, batch, scratch, scratch_bytes, own);
            e->bridge.end(st);
            return rc;
        }
    }
    std::vector<int> meta(2 * batch + 1);
    meta[0] = 0;
    bool uniform = true;
    int max_len = 0;
    for (int b = 0; b < batch; ++b) {
        ET_REQUIRE(seq_lens_host[b] >= 0, "et_encoder_run_batch: negative sequence length");
        ET_REQUIRE(!e->d_mask || seq_lens_host[b] <= e->seq_len, "et_encoder_run_batch: sequence longer than the mask");
        meta[b + 1] = meta[b] + seq_lens_host[b];
        meta[batch + 1 + b] = valid_lens_host ? valid_lens_host[b] : seq_lens_host[b];
        uniform = uniform && seq_lens_host[b] == seq_lens_host[0];
        max_len = std::max(max_len, seq_lens_host[b]);
    }
    const int T = meta[batch];
    if (T == 0) return ET_OK;
    const bool scores = e->kind == et::kLength && e->materialize_scores && uniform;
    size_t need = (size_t)5 * e->d_model * T;
    if (scores) need += (size_t)batch * e->nheads * max_len * max_len;
    ET_REQUIRE(scratch_bytes >= need * sizeof(half), "et_encoder_run_batch: scratch buffer too small");
    const int* cu = nullptr;
    const int* vl = nullptr;
    if (!uniform || valid_lens_host) {
        int rc = et::grow_lens(&e->d_lens, &e->lens_cap, 2 * batch + 1, [e] { e->drop_replays(); });
        if (rc) return rc;
        rc = et::cuda_status(cudaMemcpyAsync(e->d_lens, meta.data(), sizeof(int) * (2 * batch + 1),
                                                 cudaMemcpyHostToDevice, st), "et_encoder_run_batch: lengths upload");
        if (rc) return rc;
        if (!uniform) cu = e->d_lens;
        if (valid_lens_host) vl = e->d_lens + batch + 1;
    }
    // First call with given buffers and lengths runs directly, the second is captured into a graph, later ones
    // replay it. Skipped while the caller's stream is itself being captured.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (!e->use_graphs || cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
        return et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in),
                                   static_cast<half*>(scratch), T, cu, vl, batch, uniform ? seq_lens_host[0] : 0, st, max_len);
    std::vector<int64_t> key = {(int64_t)(intptr_t)out, (int64_t)(intptr_t)in, (int64_t)(intptr_t)scratch,
                                (int64_t)batch, (int64_t)(valid_lens_host != nullptr), (int64_t)e->materialize_scores,
                                (int64_t)(intptr_t)e->d_lens};
    for (int v : meta) key.push_back(v);
    Encoder::Replay* slot = nullptr;
    for (auto& r : e->replays)
        if (r.key == key) slot = &r;
    if (!slot) {
        if (e->replays.size() >= 8) {
            if (e->replays.front().exec) cudaGraphExecDestroy(e->replays.front().exec);
            e->replays.erase(e->replays.begin());
        }
        e->replays.push_back({key, 0, nullptr});
        slot = &e->replays.back();
    }
    if (slot->exec) return et::cuda_status(cudaGraphLaunch(slot->exec, st), "et_encoder_run_batch: graph launch");
    if (slot->seen++ == 0)
        return et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in),
                                   static_cast<half*>(scratch), T, cu, vl, batch, uniform ? seq_lens_host[0] : 0, st, max_len);
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in),
                                   static_cast<half*>(scratch), T, cu, vl, batch, uniform ? seq_lens_host[0] : 0, st, max_len);
    }
    const int frc = et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in),
                                        static_cast<half*>(scratch), T, cu, vl, batch,
                                        uniform ? seq_lens_host[0] : 0, st, max_len);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(st, &graph);
    if (frc != ET_OK || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        e->use_graphs = false;   // fall back to plain launches for this encoder
        return et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in),
                                   static_cast<half*>(scratch), T, cu, vl, batch, uniform ? seq_lens_host[0] : 0, st, max_len);
    }
    const cudaError_t ie = cudaGraphInstantiate(&slot->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        slot->exec = nullptr;
        cudaGetLastError();
        e->use_graphs = false;
        return et::encoder_forward(e, static_cast<half*>(out), static_cast<const half*>(in),
                                   static_cast<half*>(scratch), T, cu, vl, batch, uniform ? seq_lens_host[0] : 0, st, max_len);
    }
    return et::cuda_status(cudaGraphLaunch(slot->exec, st), "et_encoder_run_batch: graph launch");
}

// Reads and clears the error words of every kernel the layer launches: the tile GEMMs' (one per owned weight) and
// the current device's attention word. Synchronises.
static int encoder_check(Encoder* e, int* code) {
    std::vector<et::TileWeight*> ws(e->lin, e->lin + 6);
    ws.push_back(e->qkv);
    for (RowWeight* r : {e->rq, e->rk, e->rv})
        if (r) ws.push_back(r->tw);
    for (et::TileWeight* w : ws) {
        if (!w) continue;
        int c = 0;
        const int rc = et::tile_weight_error(w, &c);
        if (rc) return rc;
        if (c && !*code) *code = c;
    }
    int c = 0;
    const int rc = et::attention_tc_error(&c);
    if (rc) return rc;
    if (c && !*code) *code = c;
    return ET_OK;
}

int et_encoder_check(et_encoder* enc, int* code) {
    ET_REQUIRE(enc && enc->e && code, "et_encoder_check: null pointer");
    *code = 0;
    const int rc = encoder_check(enc->e, code);
    if (rc) return rc;
    if (*code) {
        et::set_error("encoder layer: device wait %d gave up", *code);
        return ET_ERR_DEVICE_TIMEOUT;
    }
    return ET_OK;
}

int et_attention_check(int* code) {
    ET_REQUIRE(code, "et_attention_check: null pointer");
    const int rc = et::attention_tc_error(code);
    if (rc) return rc;
    if (*code) {
        et::set_error("attention: device wait %d gave up", *code);
        return ET_ERR_DEVICE_TIMEOUT;
    }
    return ET_OK;
}

int et_encoder_set_graph_replay(et_encoder* enc, int on) {
    ET_REQUIRE(enc && enc->e, "et_encoder_set_graph_replay: null encoder");
    enc->e->use_graphs = on != 0;
    return ET_OK;
}


struct et_model {
    et::Model* m;
};

int et_model_create(et_model** out, et_encoder* const* layers, int n_layers) {
    ET_REQUIRE(out, "et_model_create: null output");
    *out = nullptr;
    ET_REQUIRE(layers && n_layers > 0, "et_model_create: no layers");
    for (int i = 0; i < n_layers; ++i) {
        ET_REQUIRE(layers[i] && layers[i]->e, "et_model_create: null or already consumed layer");
        ET_REQUIRE(layers[i]->e->d_model == layers[0]->e->d_model, "et_model_create: layers differ in d_model");
        for (int j = 0; j < i; ++j) ET_REQUIRE(layers[i] != layers[j], "et_model_create: the same layer twice");
    }
    auto* m = new et::Model();
    for (int i = 0; i < n_layers; ++i) {
        m->layers.push_back(layers[i]->e);
        layers[i]->e = nullptr;   // ownership moves to the model; the caller still destroys the emptied handles
    }
    *out = new et_model{m};
    return ET_OK;
}

int et_model_set_layernorm_fusion(et_model* model, int on) {
    ET_REQUIRE(model && model->m, "et_model_set_layernorm_fusion: null model");
    et::Model* m = model->m;
    m->drop_replays();
    if (!on) { m->drop_fused(); return ET_OK; }
    return et::model_prepare_fusion(m);
}

int et_model_layernorm_fused(const et_model* model) { return model && model->m && model->m->fuse_ln ? 1 : 0; }

int et_model_destroy(et_model* model) {
    if (model) { delete model->m; delete model; }
    return ET_OK;
}

int et_model_num_layers(const et_model* model) { return model && model->m ? (int)model->m->layers.size() : 0; }

int et_model_check(et_model* model, int* code) {
    ET_REQUIRE(model && model->m && code, "et_model_check: null pointer");
    *code = 0;
    for (Encoder* e : model->m->layers) {
        const int rc = encoder_check(e, code);
        if (rc) return rc;
    }
    for (const auto& f : model->m->fused)
        for (et::TileWeight* w : {f.ffn1, f.qkv}) {
            if (!w) continue;
            int c = 0;
            const int rc = et::tile_weight_error(w, &c);
            if (rc) return rc;
            if (c && !*code) *code = c;
        }
    if (*code) {
        et::set_error("layer stack: device wait %d gave up", *code);
        return ET_ERR_DEVICE_TIMEOUT;
    }
    return ET_OK;
}

int et_model_set_graph_replay(et_model* model, int on) {
    ET_REQUIRE(model && model->m, "et_model_set_graph_replay: null model");
    model->m->use_graphs = on != 0;
    return ET_OK;
}

// Grows the model's scratch to hold a batch of `total_tokens` packed tokens (and, for length layers that
// materialise scores, batch x heads x max_len^2 scores). Graphs recorded with the old scratch are dropped.
int et_model_reserve(et_model* model, int total_tokens, int batch, int max_len) {
    ET_REQUIRE(model && model->m, "et_model_reserve: null model");
    ET_REQUIRE(total_tokens >= 0 && batch >= 0 && max_len >= 0, "et_model_reserve: negative size");
    et::Model* m = model->m;
    const size_t need = et::model_scratch_halfs(m, total_tokens, batch, max_len);
    size_t need_stats = 0;
    for (const auto& f : m->fused) need_stats = std::max(need_stats, (size_t)total_tokens * std::max(f.np1, f.np2) * 2);
    if (need > m->scratch_halfs) {
        m->drop_replays();
        cudaFree(m->scratch);
        m->scratch = nullptr; m->scratch_halfs = 0;
        if (cudaMalloc(&m->scratch, need * sizeof(half)) != cudaSuccess) return et::fail(ET_ERR_CUDA, "et_model_reserve: cudaMalloc failed");
        m->scratch_halfs = need;
    }
    if (need_stats > m->stats_floats) {
        m->drop_replays();
        cudaFree(m->stats1); cudaFree(m->stats2);
        m->stats1 = m->stats2 = nullptr; m->stats_floats = 0;
        if (cudaMalloc(&m->stats1, need_stats * sizeof(float)) != cudaSuccess || cudaMalloc(&m->stats2, need_stats * sizeof(float)) != cudaSuccess)
            return et::fail(ET_ERR_CUDA, "et_model_reserve: cudaMalloc failed");
        m->stats_floats = need_stats;
    }
    return ET_OK;
}

int et_model_run_batch(et_model* model, void* out, const void* in, const int* seq_lens_host,
                       const int* valid_lens_host, int batch, void* stream) {
    ET_REQUIRE(model && model->m && out && in, "et_model_run_batch: null pointer");
    ET_REQUIRE(batch >= 0, "et_model_run_batch: negative batch");
    et::Model* m = model->m;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (batch == 0) return ET_OK;
    ET_REQUIRE(seq_lens_host, "et_model_run_batch: null seq_lens");
    if (m->use_graphs && et::StreamBridge::is_legacy(st)) {
        // the legacy default stream cannot be captured: run on the model's own stream, ordered by events
        cudaStream_t own = m->bridge.begin(st);
        if (own) {
            const int rc = et_model_run_batch(model, out, in, seq_lens_host, valid_lens_host, batch, own);
            m->bridge.end(st);
            return rc;
        }
    }
    std::vector<int> meta(2 * batch + 1);
    meta[0] = 0;
    bool uniform = true;
    int max_len = 0;
    for (int b = 0; b < batch; ++b) {
        ET_REQUIRE(seq_lens_host[b] >= 0, "et_model_run_batch: negative sequence length");
        for (Encoder* e : m->layers)
            ET_REQUIRE(!e->d_mask || seq_lens_host[b] <= e->seq_len, "et_model_run_batch: sequence longer than a layer's mask");
        meta[b + 1] = meta[b] + seq_lens_host[b];
        meta[batch + 1 + b] = valid_lens_host ? valid_lens_host[b] : seq_lens_host[b];
        uniform = uniform && seq_lens_host[b] == seq_lens_host[0];
        max_len = std::max(max_len, seq_lens_host[b]);
    }
    const int T = meta[batch];
    if (T == 0) return ET_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    const bool capturing = cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone;
    if (capturing) {
        // inside the caller's own capture nothing may be allocated or uploaded from a temporary
        size_t need_stats = 0;
        for (const auto& f : m->fused) need_stats = std::max(need_stats, (size_t)T * std::max(f.np1, f.np2) * 2);
        ET_REQUIRE(et::model_scratch_halfs(m, T, batch, max_len) <= m->scratch_halfs && need_stats <= m->stats_floats,
                   "et_model_run_batch: call et_model_reserve before capturing");
        ET_REQUIRE(uniform && !valid_lens_host, "et_model_run_batch: only equal-length batches can run inside the caller's capture");
    } else {
        int rc = et_model_reserve(model, T, batch, max_len);
        if (rc) return rc;
    }
    const int* cu = nullptr;
    const int* vl = nullptr;
    if (!uniform || valid_lens_host) {
        int rc = et::grow_lens(&m->d_lens, &m->lens_cap, 2 * batch + 1, [m] { m->drop_replays(); });
        if (rc) return rc;
        rc = et::cuda_status(cudaMemcpyAsync(m->d_lens, meta.data(), sizeof(int) * (2 * batch + 1),
                                                 cudaMemcpyHostToDevice, st), "et_model_run_batch: lengths upload");
        if (rc) return rc;
        if (!uniform) cu = m->d_lens;
        if (valid_lens_host) vl = m->d_lens + batch + 1;
    }
    half* o = static_cast<half*>(out);
    const half* x = static_cast<const half*>(in);
    const int ul = uniform ? seq_lens_host[0] : 0;
    if (!m->use_graphs || capturing) return et::model_forward(m, o, x, T, cu, vl, batch, ul, st, max_len);
    // First call with given buffers and lengths runs directly, the second is captured, later ones replay.
    std::vector<int64_t> key = {(int64_t)(intptr_t)out, (int64_t)(intptr_t)in, (int64_t)batch,
                                (int64_t)(valid_lens_host != nullptr), (int64_t)(intptr_t)m->d_lens};
    for (Encoder* e : m->layers) key.push_back((int64_t)e->materialize_scores);
    for (int v : meta) key.push_back(v);
    et::Model::Replay* slot = nullptr;
    for (auto& r : m->replays)
        if (r.key == key) slot = &r;
    if (!slot) {
        if (m->replays.size() >= 8) {
            if (m->replays.front().exec) cudaGraphExecDestroy(m->replays.front().exec);
            m->replays.erase(m->replays.begin());
        }
        m->replays.push_back({key, 0, nullptr});
        slot = &m->replays.back();
    }
    if (slot->exec) return et::cuda_status(cudaGraphLaunch(slot->exec, st), "et_model_run_batch: graph launch");
    if (slot->seen++ == 0) return et::model_forward(m, o, x, T, cu, vl, batch, ul, st, max_len);
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return et::model_forward(m, o, x, T, cu, vl, batch, ul, st, max_len);
    }
    const int frc = et::model_forward(m, o, x, T, cu, vl, batch, ul, st, max_len);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(st, &graph);
    if (frc != ET_OK || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        m->use_graphs = false;   // plain launches from now on
        return et::model_forward(m, o, x, T, cu, vl, batch, ul, st, max_len);
    }
    const cudaError_t ie = cudaGraphInstantiate(&slot->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        slot->exec = nullptr;
        cudaGetLastError();
        m->use_graphs = false;
        return et::model_forward(m, o, x, T, cu, vl, batch, ul, st, max_len);
    }
    return et::cuda_status(cudaGraphLaunch(slot->exec, st), "et_model_run_batch: graph launch");
}

}  // extern "C"
