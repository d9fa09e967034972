// Host-side interface of the tile-sparse linear (packed weight object + launch).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace et {

struct TileWeight;

// Validates the BSR arrays (host pointers), re-packs them for the kernel and uploads.
// nb_override > 0 forces the block-rows-per-CTA choice (tests); 0 picks it from size_hint.
int tile_weight_pack(TileWeight** out, int K, int N, int size_hint, long ntile, const half* data,
                     const int* row_ptr, const int* row_offset, const half* bias, int nb_override);
// New weight = the parts' output features back to back (equal in_feat); the parts stay valid.
int tile_weight_concat(TileWeight** out, const TileWeight* const* parts, int count, int size_hint);
int tile_weight_out_feat(const TileWeight* w);
void tile_weight_free(TileWeight* w);
// bias_dev != null replaces the weight's own bias for this launch (device pointer, N halfs).
int tile_linear_run(const TileWeight* w, half* Y, const half* X, int T, int gelu, cudaStream_t st,
                    const half* bias_dev = nullptr);
// Reads and clears the device error word (0 = no bounded wait gave up). Synchronises.
int tile_weight_error(const TileWeight* w, int* code);
void tile_weight_info(const TileWeight* w, int* info6);
int tile_spmm_raw(half* Y, const half* X, const int* row_ptr, const int* row_offset, const half* data,
                  int M, int N, int K, const half* bias, int gelu, cudaStream_t st);
void tile_spmm_cache_clear();
// Profiling builds (-DET_GEMM_PROFILE): device buffer of >= 1024 clock64 stamps written by CTA (0,0).
void tile_gemm_set_profile_buffer(long long* dev_buf);

// 0: shortest single launch (default); 1: least SM time per launch (several batches in flight). Applies to weights
// packed afterwards.
void tile_gemm_set_goal(int goal);

}  // namespace et
