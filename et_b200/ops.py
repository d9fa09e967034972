"""Python-side mirror of the operator and layer interface, one thin wrapper per C-ABI entry.

Tensors are torch CUDA fp16/int32 tensors; host arrays are numpy. Nothing here computes: every
function forwards to `libet_b200.so`.
"""
import ctypes

import numpy as np

from . import check, lib, ptr, stream_ptr

__all__ = [
    "skip_layernorm", "softmax_mask", "TileWeight", "tile_spmm_bias", "tile_spmm_cache_clear",
    "RowWeight", "attention_otf", "attention_prune", "qk_scores", "attention_sharedqk", "attention_batch", "attention_static_scores",
    "gen_sparse_tile_mat", "gen_sparse_row_mat", "build_head_ptr", "Encoder", "encoder_buffer_size",
    "encoder_batch_buffer_size", "KIND_TILE", "KIND_PRUNE", "KIND_LENGTH", "KIND_PRUNE_QKV",
    "Model", "attention_check", "prune_dense_to_tiles", "select_rows_magnitude", "compact_rows", "set_tuning_goal",
    "set_attention_scores_fp32", "attention_scores_fp32",
]

_i = ctypes.c_int


def skip_layernorm(in_out, skip, gamma, beta, stream=None):
    """in_out[num, size] <- LN(in_out + skip) * gamma + beta, in place."""
    num, size = in_out.shape
    check(lib().et_skip_layernorm(ptr(in_out), ptr(skip), ptr(gamma), ptr(beta), _i(num), _i(size),
                                  stream_ptr(stream)))
    return in_out


def softmax_mask(scores, mask=None, valid_len=None, stream=None):
    """scores[nmat, L, L] <- softmax(scores + mask) per row, in place."""
    nmat, L, L2 = scores.shape
    assert L == L2
    check(lib().et_softmax_mask(ptr(scores), ptr(mask), _i(nmat), _i(L),
                                _i(L if valid_len is None else valid_len), stream_ptr(stream)))
    return scores


def set_tuning_goal(goal):
    """"latency" (default): weights created afterwards are packed for the shortest single launch; "throughput": for
    the least SM time per launch (several independent batches in flight on separate streams)."""
    check(lib().et_set_tuning_goal(_i({"latency": 0, "throughput": 1}[goal])))


def set_attention_scores_fp32(on):
    """False (default): the tcgen05 attention kernel accumulates Q K^T in fp16, as the reference's kernels do; True: in
    fp32 (for models whose attention logits are large; ~1.5 times the time). Process-wide, read at launch."""
    check(lib().et_set_attention_scores_fp32(_i(1 if on else 0)))


def attention_scores_fp32():
    return bool(lib().et_attention_scores_fp32())


class TileWeight:
    """Packed, device-resident 16x16 tile-pruned weight (the reference's Linear_tile)."""

    def __init__(self, in_feat, out_feat, size, data, row_ptr, row_offset, bias=None, is_gelu=False):
        self.in_feat, self.out_feat, self.size, self.is_gelu = in_feat, out_feat, size, is_gelu
        data = np.ascontiguousarray(data, dtype=np.float16)
        row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
        row_offset = np.ascontiguousarray(row_offset, dtype=np.int32)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
        self.ntile = int(row_offset.shape[0])
        self._h = ctypes.c_void_p(0)
        check(lib().et_tile_weight_create(ctypes.byref(self._h), _i(in_feat), _i(out_feat), _i(size),
                                          _i(self.ntile), ptr(data), ptr(row_ptr), ptr(row_offset),
                                          ptr(bias)))

    def run(self, out, x, gelu=None, stream=None):
        tokens = x.shape[0]
        g = self.is_gelu if gelu is None else gelu
        check(lib().et_tile_linear(self._h, ptr(out), ptr(x), _i(tokens), _i(1 if g else 0),
                                   stream_ptr(stream)))
        return out

    def check(self):
        code = _i(0)
        check(lib().et_tile_weight_check(self._h, ctypes.byref(code)))

    def info(self):
        arr = (ctypes.c_int * 6)()
        check(lib().et_tile_weight_info(self._h, arr))
        return dict(zip(["nb", "n_chunks", "k_chunks", "stages", "stage_bytes", "packed_bytes"], arr))

    def close(self):
        if self._h:
            lib().et_tile_weight_destroy(self._h)
            self._h = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def tile_spmm_bias(Y, X, row_ptr, row_offset, data, bias, K=None, gelu=False, stream=None):
    """Launcher-level entry with device-resident tile arrays (packed form cached by address)."""
    M, N = Y.shape
    K = X.shape[1] if K is None else K
    check(lib().et_tile_spmm_bias(ptr(Y), ptr(X), ptr(row_ptr), ptr(row_offset), ptr(data), _i(M),
                                  _i(N), _i(K), ptr(bias), _i(1 if gelu else 0), stream_ptr(stream)))
    return Y


def tile_spmm_cache_clear():
    check(lib().et_tile_spmm_cache_clear())


# ---------------------------------------------------------------------------------- row-pruned linear
class RowWeight:
    """Row-pruned linear (the reference's Linear_row): only `row_id` output features are kept."""

    def __init__(self, in_feat, out_feat, size, weight, row_id, bias, nhead):
        weight = np.ascontiguousarray(weight, dtype=np.float16)
        row_id = np.ascontiguousarray(row_id, dtype=np.int32)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
        self.in_feat, self.out_feat, self.size, self.nhead = in_feat, out_feat, size, nhead
        self._h = ctypes.c_void_p(0)
        check(lib().et_row_weight_create(ctypes.byref(self._h), _i(in_feat), _i(out_feat), _i(size),
                                         ptr(weight), ptr(row_id), _i(len(row_id)), ptr(bias), _i(nhead)))
        nrow, n = _i(0), _i(0)
        rid, hp = ctypes.c_void_p(0), ctypes.c_void_p(0)
        hph = (ctypes.c_int * (nhead + 1))()
        check(lib().et_row_weight_meta(self._h, ctypes.byref(nrow), ctypes.byref(n), ctypes.byref(rid),
                                       ctypes.byref(hp), hph))
        self.nrow, self.row_id_size = nrow.value, n.value
        self.row_id_dev, self.head_ptr_dev = rid, hp          # device addresses (c_void_p)
        self.head_ptr = np.array(list(hph), dtype=np.int32)

    def run(self, out, x, stream=None):
        check(lib().et_row_linear(self._h, ptr(out), ptr(x), _i(x.shape[0]), stream_ptr(stream)))
        return out

    def close(self):
        if self._h:
            lib().et_row_weight_destroy(self._h)
            self._h = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------------- attention
def attention_otf(out, Q, K, V, mask, seq_len, d_model, nhead, stream=None):
    check(lib().et_attention_otf(ptr(out), ptr(Q), ptr(K), ptr(V), ptr(mask), _i(seq_len), _i(d_model),
                                 _i(nhead), stream_ptr(stream)))
    return out


def attention_prune(out, Q, K, V, v_col_id, v_head_ptr, nnz_col_v, mask, seq_len, d_model, nhead, stream=None):
    check(lib().et_attention_prune(ptr(out), ptr(Q), ptr(K), ptr(V), ptr(v_col_id), ptr(v_head_ptr),
                                   _i(nnz_col_v), ptr(mask), _i(seq_len), _i(d_model), _i(nhead),
                                   stream_ptr(stream)))
    return out


def qk_scores(QK, Q, K, seq_len, d_model, nhead, stream=None):
    check(lib().et_qk_scores(ptr(QK), ptr(Q), ptr(K), _i(seq_len), _i(d_model), _i(nhead), stream_ptr(stream)))
    return QK


def attention_sharedqk(out, QK, V, mask, seq_len, d_model, nhead, stream=None):
    check(lib().et_attention_sharedqk(ptr(out), ptr(QK), ptr(V), ptr(mask), _i(seq_len), _i(d_model),
                                      _i(nhead), stream_ptr(stream)))
    return out


def attention_static_scores(out, Q, K, V, mask, seq_len, d_model, nhead, stream=None):
    """et_attention_otf's result through the library's built-in score buffer: allocates nothing."""
    check(lib().et_attention_static_scores(ptr(out), ptr(Q), ptr(K), ptr(V), ptr(mask), _i(seq_len), _i(d_model),
                                           _i(nhead), stream_ptr(stream)))
    return out


def attention_check():
    """Raises EtError (ET_ERR_DEVICE_TIMEOUT) if a bounded wait of the tensor-core attention kernel gave up on the
    current device since the last check; synchronises."""
    code = _i(0)
    check(lib().et_attention_check(ctypes.byref(code)))


def attention_batch(out, Q, K, V, d_model, nhead, cu_seqlens=None, valid_lens=None, batch=1, uniform_len=0,
                    max_seq_len=0, total_tokens=None, mask=None, mask_ld=0, qk_pitch=None, v_pitch=None, qk_head_ptr=None,
                    v_col_id=None, v_head_ptr=None, stream=None):
    total = Q.shape[0] if total_tokens is None else total_tokens
    check(lib().et_attention_batch(ptr(out), ptr(Q), ptr(K), ptr(V),
                                   _i(Q.shape[1] if qk_pitch is None else qk_pitch),
                                   _i(V.shape[1] if v_pitch is None else v_pitch), ptr(qk_head_ptr),
                                   ptr(v_col_id), ptr(v_head_ptr), ptr(mask), _i(mask_ld), ptr(cu_seqlens),
                                   ptr(valid_lens), _i(batch), _i(uniform_len), _i(max_seq_len), _i(total), _i(d_model),
                                   _i(nhead), stream_ptr(stream)))
    return out


# ---------------------------------------------------------------------------------- format generators
def gen_sparse_tile_mat(nrow, ncol, sparsity, seed, bernoulli=False):
    cap = (nrow // 16) * (ncol // 16)
    row_ptr = np.zeros(nrow // 16 + 1, dtype=np.int32)
    row_offset = np.zeros(max(cap, 1), dtype=np.int32)
    n = _i(0)
    check(lib().et_gen_sparse_tile_mat(_i(nrow), _i(ncol), ctypes.c_float(sparsity), ctypes.c_uint64(seed),
                                       _i(1 if bernoulli else 0), ptr(row_ptr), ptr(row_offset), _i(cap),
                                       ctypes.byref(n)))
    return row_ptr, row_offset[:n.value].copy()


def gen_sparse_row_mat(nrow, sparsity, seed, nhead=0):
    row_id = np.zeros(nrow, dtype=np.int32)
    n = _i(0)
    check(lib().et_gen_sparse_row_mat(_i(nrow), ctypes.c_float(sparsity), ctypes.c_uint64(seed), _i(nhead),
                                      ptr(row_id), _i(nrow), ctypes.byref(n)))
    return row_id[:n.value].copy()


def build_head_ptr(row_id, nhead, out_feat):
    row_id = np.ascontiguousarray(row_id, dtype=np.int32)
    hp = np.zeros(nhead + 1, dtype=np.int32)
    check(lib().et_build_head_ptr(ptr(row_id), _i(len(row_id)), _i(nhead), _i(out_feat), ptr(hp)))
    return hp


# ---------------------------------------------------------------------------------- encoder layers
KIND_TILE, KIND_PRUNE, KIND_LENGTH, KIND_PRUNE_QKV = 0, 1, 2, 3


def encoder_buffer_size(kind, d_model, seq_len, nheads):
    f = lib().et_encoder_buffer_size
    f.restype = ctypes.c_size_t
    return int(f(_i(kind), _i(d_model), _i(seq_len), _i(nheads)))


def encoder_batch_buffer_size(kind, d_model, total_tokens, batch, max_len, nheads):
    f = lib().et_encoder_batch_buffer_size
    f.restype = ctypes.c_size_t
    return int(f(_i(kind), _i(d_model), _i(total_tokens), _i(batch), _i(max_len), _i(nheads)))


class Encoder:
    """One encoder layer (Encoder_tile / Encoder_prune / Encoder_length of the reference).

    q, k, v, o, mlp1, mlp2 are TileWeight (or RowWeight where the kind prunes rows); the encoder takes
    ownership of them. ln = (gamma1, beta1, gamma2, beta2) host arrays; mask host [seq_len, seq_len] or None;
    buffer: device scratch tensor for run() (None if only run_batch is used)."""

    def __init__(self, kind, d_model, seq_len, nheads, buffer, q, k, v, o, mlp1, mlp2, ln, mask=None):
        self.kind, self.d_model, self.seq_len, self.nheads = kind, d_model, seq_len, nheads
        self._buffer = buffer
        self._lin = (q, k, v, o, mlp1, mlp2)
        ln = [np.ascontiguousarray(a, dtype=np.float16) for a in ln]
        mask = None if mask is None else np.ascontiguousarray(mask, dtype=np.float16)
        self._h = ctypes.c_void_p(0)
        L = lib()
        common = (ptr(ln[0]), ptr(ln[1]), ptr(ln[2]), ptr(ln[3]), ptr(mask))
        if kind in (KIND_TILE, KIND_LENGTH):
            check(L.et_encoder_tile_create(ctypes.byref(self._h), _i(kind), _i(d_model), _i(seq_len), _i(nheads),
                                           ptr(buffer), q._h, k._h, v._h, o._h, mlp1._h, mlp2._h, *common))
        elif kind == KIND_PRUNE:
            check(L.et_encoder_prune_create(ctypes.byref(self._h), _i(d_model), _i(seq_len), _i(nheads),
                                            ptr(buffer), q._h, k._h, v._h, o._h, mlp1._h, mlp2._h, *common))
        elif kind == KIND_PRUNE_QKV:
            check(L.et_encoder_prune_qkv_create(ctypes.byref(self._h), _i(d_model), _i(seq_len), _i(nheads),
                                                ptr(buffer), q._h, k._h, v._h, o._h, mlp1._h, mlp2._h, *common))
        else:
            raise ValueError("unknown encoder kind")

    def run(self, out, x, stream=None):
        check(lib().et_encoder_run(self._h, ptr(out), ptr(x), stream_ptr(stream)))
        return out

    def run_batch(self, out, x, seq_lens, scratch, valid_lens=None, stream=None):
        seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
        valid = None if valid_lens is None else np.ascontiguousarray(valid_lens, dtype=np.int32)
        check(lib().et_encoder_run_batch(self._h, ptr(out), ptr(x), ptr(seq_lens), ptr(valid), _i(len(seq_lens)),
                                         ptr(scratch), ctypes.c_size_t(scratch.numel() * scratch.element_size()),
                                         stream_ptr(stream)))
        return out

    def check(self):
        """Raises EtError (ET_ERR_DEVICE_TIMEOUT) if a device-side wait of one of the layer's kernels gave up."""
        code = _i(0)
        check(lib().et_encoder_check(self._h, ctypes.byref(code)))

    def set_graph_replay(self, on):
        check(lib().et_encoder_set_graph_replay(self._h, _i(1 if on else 0)))

    def set_materialize_scores(self, on):
        check(lib().et_encoder_set_materialize_scores(self._h, _i(1 if on else 0)))

    def close(self):
        if self._h:
            lib().et_encoder_destroy(self._h)
            self._h = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Model:
    """A stack of encoder layers run back to back on packed tokens (et_model_* of the C ABI). Takes ownership of
    the layers of the `Encoder` objects given (they become empty shells). Scratch is owned by the model."""

    def __init__(self, encoders):
        self._encoders = list(encoders)
        arr = (ctypes.c_void_p * len(self._encoders))(*[e._h for e in self._encoders])
        self._h = ctypes.c_void_p(0)
        check(lib().et_model_create(ctypes.byref(self._h), arr, _i(len(self._encoders))))

    @property
    def num_layers(self):
        return int(lib().et_model_num_layers(self._h))

    def reserve(self, total_tokens, batch, max_len):
        check(lib().et_model_reserve(self._h, _i(total_tokens), _i(batch), _i(max_len)))

    def run_batch(self, out, x, seq_lens, valid_lens=None, stream=None):
        seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
        valid = None if valid_lens is None else np.ascontiguousarray(valid_lens, dtype=np.int32)
        check(lib().et_model_run_batch(self._h, ptr(out), ptr(x), ptr(seq_lens), ptr(valid), _i(len(seq_lens)),
                                       stream_ptr(stream)))
        return out

    def set_layernorm_fusion(self, on):
        check(lib().et_model_set_layernorm_fusion(self._h, _i(1 if on else 0)))

    @property
    def layernorm_fused(self):
        return bool(lib().et_model_layernorm_fused(self._h))

    def check(self):
        """Raises EtError (ET_ERR_DEVICE_TIMEOUT) if a device-side wait of one of the stack's kernels gave up."""
        code = _i(0)
        check(lib().et_model_check(self._h, ctypes.byref(code)))

    def set_graph_replay(self, on):
        check(lib().et_model_set_graph_replay(self._h, _i(1 if on else 0)))

    def close(self):
        if self._h:
            lib().et_model_destroy(self._h)
            self._h = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------------- real-weight ingestion
def prune_dense_to_tiles(weight, sparsity):
    """Dense fp16 [out_feat, in_feat] -> (row_ptr, row_offset, data[ntile, 256]) keeping the tiles of largest norm."""
    w = np.ascontiguousarray(weight, dtype=np.float16)
    out_feat, in_feat = w.shape
    cap = (out_feat // 16) * (in_feat // 16)
    row_ptr = np.zeros(out_feat // 16 + 1, dtype=np.int32)
    row_offset = np.zeros(max(cap, 1), dtype=np.int32)
    data = np.zeros((max(cap, 1), 256), dtype=np.float16)
    n = _i(0)
    check(lib().et_prune_dense_to_tiles(ptr(w), _i(out_feat), _i(in_feat), ctypes.c_float(sparsity), ptr(row_ptr),
                                        ptr(row_offset), ptr(data), _i(cap), ctypes.byref(n)))
    return row_ptr, row_offset[:n.value].copy(), data[:n.value].copy()


def select_rows_magnitude(weights, nhead, sparsity):
    """Row ids (ascending) kept per head by summed squared norm over the given dense [out_feat, in_feat] weights."""
    ws = [np.ascontiguousarray(w, dtype=np.float16) for w in weights]
    out_feat, in_feat = ws[0].shape
    arr = (ctypes.c_void_p * len(ws))(*[w.ctypes.data for w in ws])
    row_id = np.zeros(out_feat, dtype=np.int32)
    n = _i(0)
    check(lib().et_select_rows_magnitude(arr, _i(len(ws)), _i(out_feat), _i(in_feat), _i(nhead),
                                         ctypes.c_float(sparsity), ptr(row_id), _i(out_feat), ctypes.byref(n)))
    return row_id[:n.value].copy()


def compact_rows(weight, bias, row_id):
    """(weight[ceil16(n), in_feat], bias[ceil16(n)]) of the kept rows, zero padded."""
    w = np.ascontiguousarray(weight, dtype=np.float16)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float16)
    row_id = np.ascontiguousarray(row_id, dtype=np.int32)
    nrow = (len(row_id) + 15) // 16 * 16
    wc = np.zeros((nrow, w.shape[1]), dtype=np.float16)
    bc = np.zeros(nrow, dtype=np.float16)
    check(lib().et_compact_rows(ptr(w), ptr(b), _i(w.shape[0]), _i(w.shape[1]), ptr(row_id), _i(len(row_id)),
                                ptr(wc), ptr(bc)))
    return wc, bc
