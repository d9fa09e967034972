// Host-side builders of the tile-BSR and sorted-row-id pruned formats.
#pragma once
#include <cstdint>
#include <vector>

namespace et {

// bernoulli: each tile kept with probability 1-sparsity, ascending offsets inside a block-row.
// otherwise exactly floor(total*(1-sparsity)) tiles, a block-row's tiles listed in draw order.
long gen_sparse_tile_mat(int nrow, int ncol, float sparsity, uint64_t seed, bool bernoulli,
                         std::vector<int>& row_ptr, std::vector<int>& row_offset);
// exactly floor(nrow*(1-sparsity)) rows, sorted; with nhead > 0 every head keeps at least one row.
int gen_sparse_row_mat(int nrow, float sparsity, uint64_t seed, int nhead, std::vector<int>& row_id);
// head_ptr[h] = number of kept rows whose original index is below h*head_dim.
void build_head_ptr(const int* row_id, int n, int nhead, int out_feat, std::vector<int>& head_ptr);

}  // namespace et
