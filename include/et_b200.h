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
/* info[6] = {block_rows_per_cta, n_chunks, k_chunks, stages, stage_bytes, packed_bytes}. */
int et_tile_weight_info(const et_tile_weight* w, int* info);
/* Same contraction from DEVICE-resident tile arrays, K = in_feat explicit. The packed form of a
 * weight is built on its first use (device-to-host copy, synchronous) and cached by array address;
 * call et_tile_spmm_cache_clear() after changing a weight in place. Replaces
 * tile_spmm_add_bias_kernelLauncher / tile_spmm_add_bias_gelu_kernelLauncher
 * (kernels/kernels.h:13-20, kernels/linear.cu:152-167), whose missing K is the row pitch of X. */
int et_tile_spmm_bias(void* Y, const void* X, const int* W_row_ptr, const int* W_row_offset,
                      const void* W_data, int M, int N, int K, const void* bias, int gelu, void* stream);
int et_tile_spmm_cache_clear(void);

#ifdef __cplusplus
}
#endif
#endif /* ET_B200_H */
