// Host-side builders of the two pruned weight formats (product code; seeded and reproducible).
// Replaces test/tile_mat.cu:5-34, test/row_mat.cu:5-14 and the head_ptr construction of
// encoder/Linear.cu:74-88 of the reference. The reference draws its structure from an unseeded
// std::random_shuffle; here one documented generator (splitmix64, Fisher-Yates from the back,
// index = next() mod remaining) makes every structure a pure function of (shape, sparsity, seed).
#include <algorithm>
#include <cmath>
#include <numeric>
#include <vector>
#include <cuda_fp16.h>
#include "common.h"
#include "formats.h"

namespace et {

namespace {
struct SplitMix64 {
    uint64_t state;
    uint64_t next() {
        state += 0x9e3779b97f4a7c15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        return z ^ (z >> 31);
    }
    double unit() { return (double)(next() >> 11) * 0x1.0p-53; }
};
void fisher_yates(std::vector<int>& v, SplitMix64& g) {
    for (size_t n = v.size(); n > 1; --n) std::swap(v[n - 1], v[(size_t)(g.next() % n)]);
}
}  // namespace

long gen_sparse_tile_mat(int nrow, int ncol, float sparsity, uint64_t seed, bool bernoulli,
                         std::vector<int>& row_ptr, std::vector<int>& row_offset) {
    const int brs = nrow / 16, bcs = ncol / 16;
    SplitMix64 g{seed};
    row_ptr.assign(1, 0);
    row_offset.clear();
    if (bernoulli) {
        const double keep = 1.0 - (double)sparsity;
        for (int r = 0; r < brs; ++r) {
            for (int c = 0; c < bcs; ++c)
                if (g.unit() < keep) row_offset.push_back(c * 16);
            row_ptr.push_back((int)row_offset.size());
        }
        return (long)row_offset.size();
    }
    const long total = (long)brs * bcs;
    const long kept = (long)((double)total * (1.0 - (double)sparsity));
    std::vector<int> order(total);
    std::iota(order.begin(), order.end(), 0);
    fisher_yates(order, g);
    std::vector<std::vector<int>> rows(brs);
    for (long i = 0; i < kept; ++i) rows[order[i] / bcs].push_back((order[i] % bcs) * 16);
    for (int r = 0; r < brs; ++r) {
        row_offset.insert(row_offset.end(), rows[r].begin(), rows[r].end());
        row_ptr.push_back((int)row_offset.size());
    }
    return kept;
}

int gen_sparse_row_mat(int nrow, float sparsity, uint64_t seed, int nhead, std::vector<int>& row_id) {
    const int kept = (int)((double)nrow * (1.0 - (double)sparsity));
    SplitMix64 g{seed};
    std::vector<int> order(nrow);
    for (int attempt = 0; attempt < 1000; ++attempt) {
        std::iota(order.begin(), order.end(), 0);
        fisher_yates(order, g);
        row_id.assign(order.begin(), order.begin() + kept);
        std::sort(row_id.begin(), row_id.end());
        if (nhead <= 0) return kept;
        std::vector<int> per_head(nhead, 0);
        const int hd = nrow / nhead;
        for (int r : row_id) per_head[r / hd]++;
        if (std::all_of(per_head.begin(), per_head.end(), [](int c) { return c > 0; })) return kept;
    }
    return -1;
}

void build_head_ptr(const int* row_id, int n, int nhead, int out_feat, std::vector<int>& head_ptr) {
    const int hd = out_feat / nhead;
    head_ptr.assign(nhead + 1, 0);
    for (int i = 0; i < n; ++i) head_ptr[row_id[i] / hd + 1]++;
    for (int h = 0; h < nhead; ++h) head_ptr[h + 1] += head_ptr[h];
}

}  // namespace et

extern "C" int et_gen_sparse_tile_mat(int nrow, int ncol, float sparsity, uint64_t seed, int bernoulli,
                                      int* row_ptr, int* row_offset, int cap, int* ntile) {
    ET_REQUIRE(row_ptr && ntile && (row_offset || cap == 0), "et_gen_sparse_tile_mat: null pointer");
    ET_REQUIRE(nrow > 0 && ncol > 0 && nrow % 16 == 0 && ncol % 16 == 0, "et_gen_sparse_tile_mat: dimensions must be positive multiples of 16");
    ET_REQUIRE(sparsity >= 0.f && sparsity <= 1.f, "et_gen_sparse_tile_mat: sparsity outside [0,1]");
    std::vector<int> rp, ro;
    const long n = et::gen_sparse_tile_mat(nrow, ncol, sparsity, seed, bernoulli != 0, rp, ro);
    *ntile = (int)n;
    if (n > cap) return et::fail(ET_ERR_INVALID, "et_gen_sparse_tile_mat: row_offset capacity too small");
    std::copy(rp.begin(), rp.end(), row_ptr);
    std::copy(ro.begin(), ro.end(), row_offset);
    return ET_OK;
}

extern "C" int et_gen_sparse_row_mat(int nrow, float sparsity, uint64_t seed, int nhead, int* row_id,
                                     int cap, int* nkeep) {
    ET_REQUIRE(row_id && nkeep, "et_gen_sparse_row_mat: null pointer");
    ET_REQUIRE(nrow > 0 && sparsity >= 0.f && sparsity <= 1.f, "et_gen_sparse_row_mat: bad arguments");
    ET_REQUIRE(nhead <= 0 || nrow % nhead == 0, "et_gen_sparse_row_mat: nrow not divisible by nhead");
    std::vector<int> ids;
    const int n = et::gen_sparse_row_mat(nrow, sparsity, seed, nhead, ids);
    if (n < 0) return et::fail(ET_ERR_UNSUPPORTED, "et_gen_sparse_row_mat: no draw keeps a row in every head");
    *nkeep = n;
    if (n > cap) return et::fail(ET_ERR_INVALID, "et_gen_sparse_row_mat: row_id capacity too small");
    std::copy(ids.begin(), ids.end(), row_id);
    return ET_OK;
}

extern "C" int et_build_head_ptr(const int* row_id, int n, int nhead, int out_feat, int* head_ptr) {
    ET_REQUIRE(row_id && head_ptr && n >= 0 && nhead > 0 && out_feat % nhead == 0, "et_build_head_ptr: bad arguments");
    for (int i = 0; i < n; ++i)
        ET_REQUIRE(row_id[i] >= 0 && row_id[i] < out_feat && (i == 0 || row_id[i] > row_id[i - 1]),
                   "et_build_head_ptr: row_id must be strictly ascending and inside [0, out_feat)");
    std::vector<int> hp;
    et::build_head_ptr(row_id, n, nhead, out_feat, hp);
    std::copy(hp.begin(), hp.end(), head_ptr);
    return ET_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Real-weight ingestion: a dense fp16 weight [out_feat x in_feat] (row-major, host) into the two pruned formats by
// magnitude. The reference only draws random structure (test/tile_mat.cu, test/row_mat.cu) and defines no
// on-disk format; these builders produce exactly the arrays Linear_tile / Linear_row take
// (encoder/Linear.h:18-24, 66-67). Scores are sums of squares in double; ties keep the lower index, so the
// result is a pure function of the weight.
namespace et {
namespace {
double sq(const half* p, size_t n) {
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const double v = (double)__half2float(p[i]);
        s += v * v;
    }
    return s;
}
}  // namespace
}  // namespace et

extern "C" int et_prune_dense_to_tiles(const void* dense_host, int out_feat, int in_feat, float sparsity, int* row_ptr,
                                       int* row_offset, void* data, int cap_tiles, int* ntile) {
    ET_REQUIRE(dense_host && row_ptr && ntile, "et_prune_dense_to_tiles: null pointer");
    ET_REQUIRE(out_feat > 0 && in_feat > 0 && out_feat % 16 == 0 && in_feat % 16 == 0,
               "et_prune_dense_to_tiles: dimensions must be positive multiples of 16");
    ET_REQUIRE(sparsity >= 0.f && sparsity <= 1.f, "et_prune_dense_to_tiles: sparsity outside [0,1]");
    const half* W = static_cast<const half*>(dense_host);
    const int brs = out_feat / 16, bcs = in_feat / 16;
    const long total = (long)brs * bcs;
    const long kept = (long)((double)total * (1.0 - (double)sparsity));
    *ntile = (int)kept;
    if (kept > cap_tiles) return et::fail(ET_ERR_INVALID, "et_prune_dense_to_tiles: capacity too small");
    ET_REQUIRE(kept == 0 || (row_offset && data), "et_prune_dense_to_tiles: null output array");
    std::vector<double> score(total);
    for (int r = 0; r < brs; ++r)
        for (int c = 0; c < bcs; ++c) {
            double s = 0.0;
            for (int n = 0; n < 16; ++n) s += et::sq(W + (size_t)(r * 16 + n) * in_feat + c * 16, 16);
            score[(size_t)r * bcs + c] = s;
        }
    std::vector<long> order(total);
    std::iota(order.begin(), order.end(), 0L);
    std::stable_sort(order.begin(), order.end(), [&](long a, long b) { return score[a] > score[b]; });
    std::vector<char> keep(total, 0);
    for (long i = 0; i < kept; ++i) keep[order[i]] = 1;
    half* D = static_cast<half*>(data);
    long t = 0;
    row_ptr[0] = 0;
    for (int r = 0; r < brs; ++r) {
        for (int c = 0; c < bcs; ++c) {
            if (!keep[(size_t)r * bcs + c]) continue;
            row_offset[t] = c * 16;
            // data[i*256 + n*16 + k] = W[16 r + n, row_offset[i] + k]   (kernels/linear.cu:76)
            for (int n = 0; n < 16; ++n)
                std::copy(W + (size_t)(r * 16 + n) * in_feat + c * 16, W + (size_t)(r * 16 + n) * in_feat + c * 16 + 16,
                          D + (size_t)t * 256 + n * 16);
            ++t;
        }
        row_ptr[r + 1] = (int)t;
    }
    return ET_OK;
}

extern "C" int et_select_rows_magnitude(const void* const* dense_hosts, int n_mats, int out_feat, int in_feat, int nhead,
                                        float sparsity, int* row_id, int cap, int* nkeep) {
    ET_REQUIRE(dense_hosts && n_mats > 0 && row_id && nkeep, "et_select_rows_magnitude: null pointer");
    ET_REQUIRE(out_feat > 0 && in_feat > 0 && nhead > 0 && out_feat % nhead == 0, "et_select_rows_magnitude: bad dimensions");
    ET_REQUIRE(sparsity >= 0.f && sparsity <= 1.f, "et_select_rows_magnitude: sparsity outside [0,1]");
    for (int m = 0; m < n_mats; ++m) ET_REQUIRE(dense_hosts[m], "et_select_rows_magnitude: null matrix");
    const int hd = out_feat / nhead;
    // the same number of rows in every head (at least one), so that heads stay balanced
    const int per_head = std::max(1, (int)std::floor((double)hd * (1.0 - (double)sparsity) + 0.5));
    *nkeep = per_head * nhead;
    if (*nkeep > cap) return et::fail(ET_ERR_INVALID, "et_select_rows_magnitude: capacity too small");
    std::vector<double> score(out_feat, 0.0);
    for (int m = 0; m < n_mats; ++m) {
        const half* W = static_cast<const half*>(dense_hosts[m]);
        for (int r = 0; r < out_feat; ++r) score[r] += et::sq(W + (size_t)r * in_feat, in_feat);
    }
    int n = 0;
    for (int h = 0; h < nhead; ++h) {
        std::vector<int> order(hd);
        std::iota(order.begin(), order.end(), h * hd);
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return score[a] > score[b]; });
        std::sort(order.begin(), order.begin() + per_head);
        for (int i = 0; i < per_head; ++i) row_id[n++] = order[i];
    }
    return ET_OK;
}

extern "C" int et_compact_rows(const void* dense_host, const void* bias_host, int out_feat, int in_feat, const int* row_id,
                               int nkeep, void* weight_compact, void* bias_compact) {
    ET_REQUIRE(dense_host && row_id && weight_compact, "et_compact_rows: null pointer");
    ET_REQUIRE(out_feat > 0 && in_feat > 0 && nkeep >= 0 && nkeep <= out_feat, "et_compact_rows: bad dimensions");
    for (int i = 0; i < nkeep; ++i)
        ET_REQUIRE(row_id[i] >= 0 && row_id[i] < out_feat && (i == 0 || row_id[i] > row_id[i - 1]),
                   "et_compact_rows: row_id must be strictly ascending and inside [0, out_feat)");
    const half* W = static_cast<const half*>(dense_host);
    const half* B = static_cast<const half*>(bias_host);
    half* Wc = static_cast<half*>(weight_compact);
    half* Bc = static_cast<half*>(bias_compact);
    const int nrow = (nkeep + 15) / 16 * 16;   // padded with zero rows as encoder/Linear.cu:63 pads
    for (int i = 0; i < nrow; ++i) {
        if (i < nkeep) std::copy(W + (size_t)row_id[i] * in_feat, W + (size_t)(row_id[i] + 1) * in_feat, Wc + (size_t)i * in_feat);
        else std::fill(Wc + (size_t)i * in_feat, Wc + (size_t)(i + 1) * in_feat, __float2half(0.f));
        if (Bc) Bc[i] = (i < nkeep && B) ? B[row_id[i]] : __float2half(0.f);
    }
    return ET_OK;
}
