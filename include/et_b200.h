/* C ABI of the B200-native E.T. encoder hot path.
 *
 * Every function returns an int status (ET_OK = 0) and never exits the process; the text of the
 * last failure on the calling thread is available from et_last_error(). Pointers named *_host
 * are host pointers; all other data pointers are device pointers to fp16 ("half") or int32 data.
 * `stream` is a cudaStream_t passed as void* (NULL = the default stream). Work is stream-ordered
 * and no call synchronises unless its comment says so.
 *
 * Each declaration cites the interface of the reference project (cctry/E.T., paths inside that
 * project) that it stands in for.
 */
#ifndef ET_B200_H
#define ET_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ET_B200_VERSION 100

#define ET_OK 0
#define ET_ERR_INVALID 1        /* bad argument (null pointer, dimension, malformed sparse format) */
#define ET_ERR_CUDA 2           /* a CUDA runtime/driver call failed */
#define ET_ERR_UNSUPPORTED 3    /* valid but outside what the kernels cover */
#define ET_ERR_DEVICE_TIMEOUT 4 /* a bounded device-side wait gave up */

const char* et_last_error(void);
int et_version(void);

/* ---- residual add + LayerNorm -----------------------------------------------------------
 * in_out[num x size] <- LayerNorm(in_out + skip) * gamma + beta, eps 1e-6, fp32 arithmetic.
 * Replaces skip_layernorm_kernelLauncher (kernels/kernels.h:3-5, kernels/skip_layernorm.cu:101-112). */
int et_skip_layernorm(void* in_out, const void* skip, const void* gamma, const void* beta, int num,
                      int size, void* stream);

/* ---- fused additive mask + softmax over score matrices ----------------------------------
 * scores[nmat][seq_len][seq_len] <- softmax_rows(scores + mask), in place; mask [seq_len x seq_len]
 * is shared by all matrices and may be NULL; keys >= valid_len are excluded and written as 0.
 * Replaces the mask + softmax stage of sharedQK_attention_kernelLauncher (kernels/attention.cu:291-323)
 * and softmax_blk (kernels/attention.cu:10-48). */
int et_softmax_mask(void* scores, const void* mask, int nmat, int seq_len, int valid_len, void* stream);

/* ---- tile-pruned linear ------------------------------------------------------------------
 * Weight object built from HOST arrays in the reference's 16x16 tile format: row_ptr[out_feat/16+1],
 * row_offset[ntile] (input-feature offset of each kept tile, a multiple of 16),
 * data[ntile*256] with data[i*256 + n*16 + k] = W[16*r + n][row_offset[i] + k], bias[out_feat]
 * (NULL = zeros). Arrays are validated and copied; `size` is the expected token count (a hint).
 * Synchronises the device once. Replaces Linear_tile::Linear_tile (encoder/Linear.h:18-24). */
typedef struct et_tile_weight et_tile_weight;
int et_tile_weight_create(et_tile_weight** out, int in_feat, int out_feat, int size, int ntile,
                          const void* data_host, const int* row_ptr_host,
                          const int* row_offset_host, const void* bias_host);
int et_tile_weight_destroy(et_tile_weight* w);
/* Y[tokens x out_feat] = X[tokens x in_feat] . W^T + bias, tanh-GELU when gelu != 0.
 * Replaces Linear_tile::run (encoder/Linear.h:36-45). */
int et_tile_linear(const et_tile_weight* w, void* Y, const void* X, int tokens, int gelu, void* stream);
/* Reads and clears the weight's device error word (synchronises): ET_ERR_DEVICE_TIMEOUT and the
 * code in *code when a bounded wait inside the kernel gave up since the last check. */
int et_tile_weight_check(const et_tile_weight* w, int* code);
/* Extension (no counterpart in the reference): what weights created AFTERWARDS are packed for. 0 (default): the
 * shortest duration of one launch on an otherwise idle GPU (tiles spread over as many SMs as possible). 1: the
 * least SM time per launch (fewer, larger tiles), for callers that keep several independent batches in flight on
 * separate streams, where all SMs are busy anyway. Process-wide. */
#define ET_GOAL_LATENCY 0
#define ET_GOAL_THROUGHPUT 1
int et_set_tuning_goal(int goal);
/* Extension: how the tcgen05 attention kernel accumulates Q K^T. 0 (default): in fp16, as the reference's kernels
 * accumulate their scores (kernels/attention.cu:82, `c_t<half>`); the error against exact arithmetic grows with the
 * size of the scores (worst output element: 2e-3 for |q.k| up to 50, 1.4e-2 up to 165, 3e-2 up to 390). 1: in fp32
 * (2e-3 throughout, ~1.5 times the time). Process-wide, read when a launch is issued: graphs recorded earlier by
 * et_encoder_run_batch / et_model_run_batch keep the kernel they were recorded with. */
int et_set_attention_scores_fp32(int on);
int et_attention_scores_fp32(void);
/* info[6] = {block_rows_per_cta, n_chunks, k_chunks, stages, stage_bytes, packed_bytes}. */
int et_tile_weight_info(const et_tile_weight* w, int* info);
/* Same contraction from DEVICE-resident tile arrays, K = in_feat explicit. The packed form of a
 * weight is built on its first use (device-to-host copy, synchronous: not inside a stream capture) and cached
 * by the three array addresses, N and K; the bias is read from the caller's pointer at every call. Call
 * et_tile_spmm_cache_clear() after changing a weight in place AND after freeing one: a new weight of the same
 * shape that the allocator places at the same addresses would otherwise be served the old packed copy
 * (objects that own their weight, et_tile_weight_create / Linear_tile, have no such hazard). Replaces
 * tile_spmm_add_bias_kernelLauncher / tile_spmm_add_bias_gelu_kernelLauncher
 * (kernels/kernels.h:13-20, kernels/linear.cu:152-167), whose missing K is the row pitch of X. */
int et_tile_spmm_bias(void* Y, const void* X, const int* W_row_ptr, const int* W_row_offset,
                      const void* W_data, int M, int N, int K, const void* bias, int gelu, void* stream);
int et_tile_spmm_cache_clear(void);

/* ---- row-pruned linear ---------------------------------------------------------------------
 * Only row_id_size output features are kept; row_id_host[] holds their original indices, strictly
 * ascending; weight_host is the compact [row_id_size x in_feat] matrix, bias_host[row_id_size] (NULL =
 * zeros). The output has nrow = row_id_size rounded up to 16 columns (zero beyond row_id_size).
 * head_ptr[h] = number of kept rows below h*(out_feat/nhead), h = 0..nhead.
 * Replaces Linear_row::Linear_row (encoder/Linear.h:66-67, encoder/Linear.cu:60-91). */
typedef struct et_row_weight et_row_weight;
int et_row_weight_create(et_row_weight** out, int in_feat, int out_feat, int size, const void* weight_host,
                         const int* row_id_host, int row_id_size, const void* bias_host, int nhead);
int et_row_weight_destroy(et_row_weight* w);
/* out[tokens x nrow] = in . W^T + bias. Replaces Linear_row::run (encoder/Linear.h:68-71) and
 * row_spmm_add_bias_kernelLauncher (kernels/kernels.h:7-11, kernels/linear.cu:18-34); no cuBLAS handle. */
int et_row_linear(const et_row_weight* w, void* out, const void* in, int tokens, void* stream);
/* Same contraction from a DEVICE-resident dense compact weight [N x K], N and K multiples of 16 (the
 * reference pads N to 16): out[M x N] = in[M x K] . weight^T + bias. Packed on first use and cached by
 * weight address, N and K, with the same address-reuse hazard as et_tile_spmm_bias (et_tile_spmm_cache_clear
 * drops the cache); the bias is read from the caller's pointer at every call. Replaces row_spmm_add_bias_kernelLauncher
 * (kernels/kernels.h:7-11, kernels/linear.cu:18-34) without its cuBLAS handle and algorithm. */
int et_row_spmm_bias(void* out, const void* in, const void* weight, const void* bias, int M, int N, int K,
                     void* stream);
/* The public members of Linear_row that the encoder reads (encoder/encoder.cu:76-79): any of the
 * output pointers may be NULL. head_ptr_host receives nhead+1 ints. */
int et_row_weight_meta(const et_row_weight* w, int* nrow, int* row_id_size, const int** row_id_dev,
                       const int** head_ptr_dev, int* head_ptr_host);

/* ---- attention --------------------------------------------------------------------------------
 * out[seq_len x d_model], head h in columns [h*hd, (h+1)*hd): softmax(Q_h K_h^T / sqrt(hd) + mask) V_h.
 * mask: additive [seq_len x seq_len] fp16 shared by all heads, or NULL. Any seq_len >= 0.
 * Replaces OTF_attention_kernelLauncher (kernels/kernels.h:22-24, kernels/attention.cu:122-134). */
int et_attention_otf(void* out, const void* Q, const void* K, const void* V, const void* mask, int seq_len,
                     int d_model, int nhead, void* stream);
/* V compact [seq_len x nnz_col_v]; head h owns compact columns [v_head_ptr[h], v_head_ptr[h+1]); result
 * column j is stored at out column v_col_id[j], every other out column is written as 0.
 * Replaces Prune_attention_kernelLauncher (kernels/kernels.h:26-30, kernels/attention.cu:252-271). */
int et_attention_prune(void* out, const void* Q, const void* K, const void* V, const int* v_col_id,
                       const int* v_head_ptr, int nnz_col_v, const void* mask, int seq_len, int d_model,
                       int nhead, void* stream);
/* QK[nhead][seq_len][seq_len] = Q_h K_h^T / sqrt(hd), Q and K with row pitch d_model.
 * Replaces the cublasHgemmStridedBatched call of Encoder_length::run (encoder/encoder.cu:126-130). */
int et_qk_scores(void* QK, const void* Q, const void* K, int seq_len, int d_model, int nhead, void* stream);
/* out = softmax(QK + mask) V per head from precomputed scores.
 * Replaces sharedQK_attention_kernelLauncher (kernels/kernels.h:32-34, kernels/attention.cu:342-350). */
int et_attention_sharedqk(void* out, const void* QK, const void* V, const void* mask, int seq_len,
                          int d_model, int nhead, void* stream);
/* Attention for callers that cannot allocate device memory (no counterpart in the reference). Same
 * arguments and result as et_attention_otf, computed through score matrices kept in an 8 MiB device array
 * that is part of the library image, so the call allocates nothing: not with cudaMalloc and not through
 * any library. Meant for hosts with a fixed memory plan (a real-time loop, a plugin whose host process
 * owns the allocator). Limit: nhead * seq_len * seq_len <= 16 * 512 * 512, otherwise ET_ERR_UNSUPPORTED.
 * The first call on each device looks up the array's device address; make that call before any stream
 * capture starts. All calls on a device share the array: issue them on one stream, calls that overlap
 * on the GPU race. Nothing needs clearing between calls. */
int et_attention_static_scores(void* out, const void* Q, const void* K, const void* V, const void* mask,
                               int seq_len, int d_model, int nhead, void* stream);
/* Reads and clears the current device's error word of the tensor-core attention kernel (synchronises):
 * ET_ERR_DEVICE_TIMEOUT and the code in *code (21: the issuing thread's wait, 22: the final accumulator wait)
 * when a bounded wait inside the kernel gave up since the last check; the rows of that CTA are then not
 * written. The word is one per device, shared by every launch on it. No counterpart in the reference, whose
 * only error handling is cudaChk's exit(1) (encoder/utils.h:4-12). */
int et_attention_check(int* code);
/* Batched, variable-length form (no counterpart in the reference, which handles one sequence per call):
 * sequences are packed back to back; cu_seqlens (device, batch+1 ints) gives their token offsets, or NULL
 * for `batch` sequences of uniform_len tokens. valid_lens (device, may be NULL) excludes keys at or beyond
 * valid_lens[b] (key padding). Q and K share qk_pitch; qk_head_ptr / v_head_ptr + v_col_id (device, may be
 * NULL) select compact per-head column windows as in et_attention_prune. max_seq_len: the longest sequence
 * when cu_seqlens is given (0 = unknown); it only selects between the tensor-core kernel for dense heads of
 * 64 with at most 512 keys and the general kernel. */
int et_attention_batch(void* out, const void* Q, const void* K, const void* V, int qk_pitch, int v_pitch,
                       const int* qk_head_ptr, const int* v_col_id, const int* v_head_ptr, const void* mask,
                       int mask_ld, const int* cu_seqlens, const int* valid_lens, int batch, int uniform_len,
                       int max_seq_len, int total_tokens, int d_model, int nhead, void* stream);

/* ---- pruned-format generators (host) ----------------------------------------------------------
 * Seeded and reproducible. bernoulli == 0 keeps exactly floor(total*(1-sparsity)) tiles (a block-row's
 * tiles in draw order); otherwise each tile is kept with probability 1-sparsity (ascending offsets).
 * Replaces gen_sparse_tile_mat (test/tile_mat.cu:5-34) and gen_sparse_row_mat (test/row_mat.cu:5-14). */
int et_gen_sparse_tile_mat(int nrow, int ncol, float sparsity, uint64_t seed, int bernoulli, int* row_ptr,
                           int* row_offset, int cap, int* ntile);
int et_gen_sparse_row_mat(int nrow, float sparsity, uint64_t seed, int nhead, int* row_id, int cap, int* nkeep);
int et_build_head_ptr(const int* row_id, int n, int nhead, int out_feat, int* head_ptr);

/* ---- real-weight ingestion (host; extension) ------------------------------------------------------
 * The reference only draws random structure (test/tile_mat.cu, test/row_mat.cu) and defines no on-disk format.
 * These turn a dense fp16 weight [out_feat x in_feat] (row-major) into exactly the arrays Linear_tile
 * (encoder/Linear.h:18-24) and Linear_row (encoder/Linear.h:66-67) take, by magnitude; ties keep the lower
 * index, so the result is a pure function of the weight.
 * et_prune_dense_to_tiles: keeps the floor(total*(1-sparsity)) 16x16 tiles of largest sum of squares; tiles of a
 *   block-row in ascending column order; data[i*256 + n*16 + k] = W[16r+n, row_offset[i]+k].
 * et_select_rows_magnitude: per head keeps the round(head_dim*(1-sparsity)) (at least 1) rows of largest sum of
 *   squares, summed over the n_mats matrices given (pass Q and K together so that they retain the same
 *   dimensions); row_id ascending.
 * et_compact_rows: weight_compact [ceil16(nkeep) x in_feat] (zero rows as padding), bias_compact [ceil16(nkeep)]. */
int et_prune_dense_to_tiles(const void* dense_host, int out_feat, int in_feat, float sparsity, int* row_ptr,
                            int* row_offset, void* data, int cap_tiles, int* ntile);
int et_select_rows_magnitude(const void* const* dense_hosts, int n_mats, int out_feat, int in_feat, int nhead,
                             float sparsity, int* row_id, int cap, int* nkeep);
int et_compact_rows(const void* dense_host, const void* bias_host, int out_feat, int in_feat, const int* row_id,
                    int nkeep, void* weight_compact, void* bias_compact);

/* ---- encoder layers ----------------------------------------------------------------------------
 * One post-LN encoder layer: Q,K,V linears -> attention -> output linear -> add+LayerNorm -> MLP1 (GELU)
 * -> MLP2 -> add+LayerNorm (encoder/encoder.cu:20-45). LayerNorm vectors (d_model) and mask
 * (seq_len x seq_len additive, may be NULL) are HOST pointers and are copied; `buffer` is a DEVICE
 * scratch of et_encoder_buffer_size bytes owned by the caller (may be NULL if only run_batch is used).
 * The encoder takes ownership of the linears passed in (their handles stay valid only for destroy),
 * as the reference's constructors take them by rvalue. kind: 0 = Encoder_tile, 2 = Encoder_length
 * (encoder/encoder.h:56-77, :102-134). */
typedef struct et_encoder et_encoder;
int et_encoder_tile_create(et_encoder** out, int kind, int d_model, int seq_len, int nheads, void* buffer,
                           et_tile_weight* q, et_tile_weight* k, et_tile_weight* v, et_tile_weight* o,
                           et_tile_weight* mlp1, et_tile_weight* mlp2, const void* ln_gamma_1,
                           const void* ln_beta_1, const void* ln_gamma_2, const void* ln_beta_2,
                           const void* mask_host);
/* Encoder_prune (encoder/encoder.h:79-100): V is row-pruned. */
int et_encoder_prune_create(et_encoder** out, int d_model, int seq_len, int nheads, void* buffer,
                            et_tile_weight* q, et_tile_weight* k, et_row_weight* v, et_tile_weight* o,
                            et_tile_weight* mlp1, et_tile_weight* mlp2, const void* ln_gamma_1,
                            const void* ln_beta_1, const void* ln_gamma_2, const void* ln_beta_2,
                            const void* mask_host);
/* Extension: Q, K and V all row-pruned; Q and K must keep the same rows per head. */
int et_encoder_prune_qkv_create(et_encoder** out, int d_model, int seq_len, int nheads, void* buffer,
                                et_row_weight* q, et_row_weight* k, et_row_weight* v, et_tile_weight* o,
                                et_tile_weight* mlp1, et_tile_weight* mlp2, const void* ln_gamma_1,
                                const void* ln_beta_1, const void* ln_gamma_2, const void* ln_beta_2,
                                const void* mask_host);
int et_encoder_destroy(et_encoder* enc);
/* Encoder_base::buffer_size / Encoder_length::buffer_size (encoder/encoder.h:51-53, :129-133), in bytes. */
size_t et_encoder_buffer_size(int kind, int d_model, int seq_len, int nheads);
size_t et_encoder_batch_buffer_size(int kind, int d_model, int total_tokens, int batch, int max_len, int nheads);
/* Encoder_*::run(out, in) (encoder/encoder.h:76): one sequence of seq_len tokens; out may alias in. */
int et_encoder_run(et_encoder* enc, void* out, const void* in, void* stream);
/* Extension: a batch of packed sequences, seq_lens_host[batch] tokens each (any length >= 0, at most
 * seq_len when the encoder has a mask); valid_lens_host (may be NULL) marks keys at or beyond it as padding.
 * scratch: device buffer of et_encoder_batch_buffer_size bytes. */
int et_encoder_run_batch(et_encoder* enc, void* out, const void* in, const int* seq_lens_host,
                         const int* valid_lens_host, int batch, void* scratch, size_t scratch_bytes, void* stream);
/* Reads and clears the error words of every kernel the layer launches (its tile GEMMs and the device's
 * attention word, see et_attention_check); synchronises. ET_ERR_DEVICE_TIMEOUT with the first code found in
 * *code when a bounded device-side wait gave up since the last check: the output of that run is then
 * incomplete. The status a caller reads where the reference would have exited (encoder/utils.h:4-12). */
int et_encoder_check(et_encoder* enc, int* code);
/* et_encoder_run_batch replays a CUDA graph of the layer's launches from the third call on with the same
 * buffers and lengths (no counterpart in the reference, whose run() blocks the host three times per layer).
 * on = 0 turns that off (plain launches every call). It is skipped by itself while the caller's stream is
 * being captured. */
int et_encoder_set_graph_replay(et_encoder* enc, int on);
/* Length encoder only: route attention through scores materialised in HBM (the reference's structure,
 * encoder/encoder.cu:126-136) instead of the default on-the-fly kernel. Equal-length batches only. */
int et_encoder_set_materialize_scores(et_encoder* enc, int on);

/* ---- Stack of encoder layers (extension: no counterpart in the reference, whose objects hold one layer and
 * whose callers run it once, test/tile_test.cu:36-41). The model takes ownership of the layers (the caller still
 * calls et_encoder_destroy on the emptied handles), owns its scratch (et_model_reserve, or grown on demand by
 * et_model_run_batch outside stream capture), and from the third call with the same buffers and lengths replays
 * all launches of all layers as one CUDA graph. `out` may alias `in`. Layers may be of different kinds; they
 * must agree in d_model. */
typedef struct et_model et_model;
int et_model_create(et_model** out, et_encoder* const* layers, int n_layers);
int et_model_destroy(et_model* model);
int et_model_num_layers(const et_model* model);
int et_model_reserve(et_model* model, int total_tokens, int batch, int max_len);
int et_model_run_batch(et_model* model, void* out, const void* in, const int* seq_lens_host,
                       const int* valid_lens_host, int batch, void* stream);
int et_model_set_graph_replay(et_model* model, int on);
/* Optional form of a stack of tile / length layers: the residual-add + LayerNorm steps (encoder/encoder.cu:36-44)
 * folded into the neighbouring linears, 5 launches per layer instead of 7 (the output projection and FFN2 add the
 * residual and leave per-row sums, the next linear normalises in its epilogue with gamma folded into its weights,
 * one plain LayerNorm ends the stack). OFF by default: on B200 the longer epilogues cost more than the two
 * bandwidth-bound LayerNorm passes they replace (measured: 86 ms against 75 ms per step of the 24-layer BERT-large
 * workload). Results differ from the default form by fp16 rounding of different intermediates, within the library's
 * tolerance. on = 1 builds the folded weights (host work, synchronises); stacks with a row-pruned layer stay
 * unfused; et_model_layernorm_fused tells which form is active. */
int et_model_set_layernorm_fusion(et_model* model, int on);
int et_model_layernorm_fused(const et_model* model);
/* et_encoder_check over every layer of the stack (encoder/utils.h:4-12 is the reference's error path). */
int et_model_check(et_model* model, int* code);

#ifdef __cplusplus
}
#endif
#endif /* ET_B200_H */
