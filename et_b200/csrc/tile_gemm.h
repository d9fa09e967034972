// Host-side interface of the tile-sparse linear (packed weight object + launch).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace et {

struct TileWeight;

// LayerNorm folded into the epilogue of a tile linear (the layer stack's fused path).
//   mode 1: the input is un-normalised; its per-row partial sums stats_in[T][np_in][2] (sum, sum of squares over the
//           producer's column chunks) give mean and 1/std, applied in the epilogue; the weight must have been folded
//           with the LayerNorm's gamma / beta (tile_weight_fold).
//   mode 2: Y = X W^T + bias + resid (resid fp16 [T x N]); per-row partial sums of Y to stats_out[T][np_out][2],
//           np_out = tile_weight_stat_slots(weight).
//   mode 3: the same with resid = LayerNorm(row of `resid`) from stats_src / gamma_s / beta_s (fp32 [N]).
struct GemmFusion {
    int mode = 0;
    const float* stats_in = nullptr; int np_in = 0;
    const half* resid = nullptr;
    const float* stats_src = nullptr; int np_src = 0;
    const float* gamma_s = nullptr; const float* beta_s = nullptr;
    float* stats_out = nullptr; int np_out = 0;
    float eps = 1e-6f;
    // filled in by tile_linear_run
    const float* colc = nullptr; const float* cold = nullptr; const float* bias_f32 = nullptr;
    float inv_d_in = 0.f, inv_d_src = 0.f;
};

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
                    const half* bias_dev = nullptr, const GemmFusion* fusion = nullptr);
// New weight = w with gamma multiplied into its input features and the column vectors c_n = sum_k gamma_k W_nk,
// d_n = sum_k beta_k W_nk + bias_n that the mode-1 epilogue needs (gamma, beta: host, in_feat values).
int tile_weight_fold(TileWeight** out, const TileWeight* w, const half* gamma, const half* beta);
// Column chunks of the packed weight, and the partial-sum slots per row that its residual epilogue writes.
int tile_weight_chunks(const TileWeight* w);
int tile_weight_stat_slots(const TileWeight* w);
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
