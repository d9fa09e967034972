"""Python-side mirror of the operator and layer interface, one thin wrapper per C-ABI entry.

Tensors are torch CUDA fp16/int32 tensors; host arrays are numpy. Nothing here computes: every
function forwards to `libet_b200.so`.
"""
import ctypes

import numpy as np

from . import check, lib, ptr, stream_ptr

__all__ = [
    "skip_layernorm", "softmax_mask", "TileWeight", "tile_spmm_bias", "tile_spmm_cache_clear",
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
