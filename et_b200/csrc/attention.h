// Host-side launchers of the attention kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace et {

// General form. Q/K share q_pitch; scores != null replaces Q K^T by precomputed, already scaled
// scores [batch][nhead][L][L] (equal-length sequences only). cu_seqlens (device, batch+1 ints) or, when
// null, `batch` sequences of uniform_len tokens each. valid_lens (device) limits the keys per sequence.
// max_len: the longest sequence of the batch when the caller knows it (0 = unknown); it only selects the kernel.
int attention_launch(half* Z, const half* Q, const half* K, const half* V, const half* scores,
                     int q_pitch, int v_pitch, const int* qk_head_ptr, const int* v_col_id,
                     const int* v_head_ptr, const half* mask, int mask_ld, const int* cu_seqlens,
                     const int* valid_lens, int batch, int uniform_len, int total_tokens, int d_model,
                     int nhead, cudaStream_t st, int max_len = 0);
// tcgen05 fast path (dense, head_dim 64, longest sequence known); ET_ERR_UNSUPPORTED outside its range.
int attention_tc_launch(half* Z, const half* Q, const half* K, const half* V, int q_pitch, int v_pitch,
                        const half* mask, int mask_ld, const int* cu_seqlens, const int* valid_lens, int batch,
                        int uniform_len, int total_tokens, int max_len, int d_model, int nhead, cudaStream_t st);
// Reads and clears the current device's error word of the tcgen05 kernel's bounded waits (synchronises).
int attention_tc_error(int* code);
// One-time per-device set-up of that error word (no allocation); safe to call repeatedly.
int attention_prepare_device();
// pitch: row pitch of Q and K in elements (0 = d_model).
int qk_scores_launch(half* S, const half* Q, const half* K, int batch, int L, int d_model, int nhead,
                     cudaStream_t st, int pitch = 0);

// dst[o][t][p] = inv[o][p] >= 0 ? src[o][t][inv[o][p]] : 0 for n <= 3 operands in one launch: compact row-pruned
// activations back at their original feature positions, zeros elsewhere (d a multiple of 8).
int expand_rows_launch(int n, const half* const* src, const int* src_pitch, half* const* dst, const int* dst_pitch,
                       const int* const* inv, int d, int T, cudaStream_t st);

// Same result as the on-the-fly form for one sequence, through scores held in a device array that is part
// of the library image (no allocation). seq_len*seq_len*nhead is limited to 16*512*512.
int attention_static_scores(half* Z, const half* Q, const half* K, const half* V, const half* mask, int seq_len,
                            int d_model, int nhead, cudaStream_t st);

}  // namespace et
