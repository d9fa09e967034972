// Host-side builders of the two pruned weight formats (product code; seeded and reproducible).
// Replaces test/tile_mat.cu:5-34, test/row_mat.cu:5-14 and the head_ptr construction of
// encoder/Linear.cu:74-88 of the reference. The reference draws its structure from an unseeded
// std::random_shuffle; here one documented generator (splitmix64, Fisher-Yates from the back,
// index = next() mod remaining) makes every structure a pure function of (shape, sparsity, seed).
#include <algorithm>
#include <numeric>
#include <vector>
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
