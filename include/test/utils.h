// Builders of pruned linears for drivers and benchmarks, with the names and signatures of the reference's
// test helpers (test/utils.h:25-38, test/gen_linear.cu:5-25). Structure comes from the library's seeded
// generators; values follow the reference's fixtures (weights and biases 0.1, row weights 1.0) unless a
// standard deviation is set, in which case kept weights are N(0, std) from a seeded generator.
#pragma once
#include <cmath>
#include <cstdint>
#include <vector>
#include "../encoder/Linear.h"

namespace et_test {
inline uint64_t& seed() {
    static uint64_t s = 1234;
    return s;
}
inline float& weight_std() {   // 0 selects the reference's constant fixtures
    static float s = 0.f;
    return s;
}
inline bool& bernoulli() {     // false: exactly floor(total*(1-sparsity)) tiles, as the reference
    static bool b = false;
    return b;
}
inline uint64_t next_seed() { return seed() += 0x9e3779b97f4a7c15ull; }
inline float gaussian(uint64_t& state) {
    auto u = [&state]() {
        state += 0x9e3779b97f4a7c15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        z ^= z >> 31;
        return ((double)(z >> 11) + 0.5) * 0x1.0p-53;
    };
    return (float)(std::sqrt(-2.0 * std::log(u())) * std::cos(6.283185307179586 * u()));
}
inline void fill(std::vector<half>& v, float constant, uint64_t sd) {
    if (weight_std() <= 0.f) {
        for (auto& x : v) x = __float2half(constant);
    } else {
        for (auto& x : v) x = __float2half(weight_std() * gaussian(sd));
    }
}
}  // namespace et_test

inline void gen_sparse_tile_mat(int nrow, int ncol, float sparsity, std::vector<int>& row_ptr,
                                std::vector<int>& row_offset) {
    const int cap = (nrow / 16) * (ncol / 16);
    row_ptr.assign(nrow / 16 + 1, 0);
    row_offset.assign(cap > 0 ? cap : 1, 0);
    int ntile = 0;
    et_shim::require_ok(et_gen_sparse_tile_mat(nrow, ncol, sparsity, et_test::next_seed(), et_test::bernoulli() ? 1 : 0,
                                               row_ptr.data(), row_offset.data(), cap, &ntile),
                        "gen_sparse_tile_mat");
    row_offset.resize(ntile);
}

inline void gen_sparse_row_mat(int nrow, int ncol, float sparsity, std::vector<half>& rows, std::vector<int>& row_id,
                               int nhead = 0) {
    row_id.assign(nrow, 0);
    int keep = 0;
    et_shim::require_ok(et_gen_sparse_row_mat(nrow, sparsity, et_test::next_seed(), nhead, row_id.data(), nrow, &keep),
                        "gen_sparse_row_mat");
    row_id.resize(keep);
    rows.assign((size_t)ncol * keep, __float2half(0.f));
    et_test::fill(rows, 1.0f, et_test::next_seed());
}

inline Linear_tile gen_tile_linear(int in_feat, int out_feat, int size, float sparsity, bool is_gelu = false) {
    std::vector<int> row_ptr, row_offset;
    gen_sparse_tile_mat(out_feat, in_feat, sparsity, row_ptr, row_offset);
    std::vector<half> data(row_offset.size() * 256), bias(out_feat);
    et_test::fill(data, 0.1f, et_test::next_seed());
    for (auto& b : bias) b = __float2half(et_test::weight_std() > 0.f ? 0.f : 0.1f);
    return Linear_tile(in_feat, out_feat, size, (int)row_offset.size(), data.data(), row_ptr.data(),
                       row_offset.data(), bias.data(), is_gelu);
}

inline Linear_row gen_row_linear(int in_feat, int out_feat, int size, float sparsity, int nhead) {
    std::vector<half> rows;
    std::vector<int> row_id;
    gen_sparse_row_mat(out_feat, in_feat, sparsity, rows, row_id, nhead);
    std::vector<half> bias(row_id.size(), __float2half(et_test::weight_std() > 0.f ? 0.f : 0.1f));
    return Linear_row(in_feat, out_feat, size, rows.data(), row_id.data(), (int)row_id.size(), bias.data(), nhead);
}
