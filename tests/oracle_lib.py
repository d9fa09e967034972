"""ctypes access to the CPU oracle (oracle/liborc.so) and to the reference project's CUDA kernels
(oracle/_ref/libet_ref.so). Test infrastructure: only tests, the smoke check and the bench's
baseline legs import this module."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORC_DIR = os.path.join(ROOT, "oracle")
ORC_LIB = os.path.join(ORC_DIR, "liborc.so")
REF_LIB = os.path.join(ORC_DIR, "_ref", "libet_ref.so")

REF_COMPAT = 1

_f = ctypes.POINTER(ctypes.c_float)
_ip = ctypes.POINTER(ctypes.c_int)


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f)


def _ipp(a):
    return None if a is None else a.ctypes.data_as(_ip)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.orc_h2f.restype = ctypes.c_float
        lib.orc_h2f.argtypes = [ctypes.c_uint16]
        lib.orc_f2h.restype = ctypes.c_uint16
        lib.orc_f2h.argtypes = [ctypes.c_float]

    def threads(self):
        return int(self.lib.orc_threads())

    def gen_sparse_tile_mat(self, nrow, ncol, sparsity, seed, bernoulli=False):
        cap = (nrow // 16) * (ncol // 16)
        row_ptr = np.zeros(nrow // 16 + 1, dtype=np.int32)
        row_offset = np.zeros(max(cap, 1), dtype=np.int32)
        n = self.lib.orc_gen_sparse_tile_mat(nrow, ncol, ctypes.c_float(sparsity),
                                             ctypes.c_uint64(seed), int(bernoulli), _ipp(row_ptr),
                                             _ipp(row_offset), cap)
        assert n >= 0
        return row_ptr, row_offset[:n].copy()

    def gen_sparse_row_mat(self, nrow, sparsity, seed, nhead=0):
        row_id = np.zeros(nrow, dtype=np.int32)
        n = self.lib.orc_gen_sparse_row_mat(nrow, ctypes.c_float(sparsity), ctypes.c_uint64(seed),
                                            nhead, _ipp(row_id), nrow)
        assert n >= 0
        return row_id[:n].copy()

    def head_ptr(self, row_id, nhead, out_feat):
        hp = np.zeros(nhead + 1, dtype=np.int32)
        row_id = i32(row_id)
        self.lib.orc_head_ptr(_ipp(row_id), len(row_id), nhead, out_feat, _ipp(hp))
        return hp

    def bsr_to_dense(self, row_ptr, row_offset, data, N, K):
        W = np.zeros((N, K), dtype=np.float32)
        row_ptr, row_offset, data = i32(row_ptr), i32(row_offset), f32(data)
        self.lib.orc_bsr_to_dense(_fp(W), _ipp(row_ptr), _ipp(row_offset), _fp(data), N, K)
        return W

    def tile_linear(self, X, row_ptr, row_offset, data, bias, N, gelu=False):
        X = f32(X)
        T, K = X.shape
        Y = np.zeros((T, N), dtype=np.float32)
        row_ptr, row_offset, data = i32(row_ptr), i32(row_offset), f32(data)
        bias = None if bias is None else f32(bias)
        self.lib.orc_tile_linear(_fp(Y), _fp(X), _ipp(row_ptr), _ipp(row_offset), _fp(data),
                                 _fp(bias), T, N, K, int(gelu))
        return Y

    def row_linear(self, X, weight, bias, out_pitch=None):
        X, weight = f32(X), f32(weight)
        T, K = X.shape
        nkeep = weight.shape[0]
        out_pitch = nkeep if out_pitch is None else out_pitch
        out = np.zeros((T, out_pitch), dtype=np.float32)
        bias = None if bias is None else f32(bias)
        self.lib.orc_row_linear(_fp(out), _fp(X), _fp(weight), _fp(bias), T, nkeep, K, out_pitch)
        return out

    def attention(self, Q, K, V, seq_lens, d_model, nhead, mask=None, valid_lens=None,
                  qk_head_ptr=None, v_col_id=None, v_head_ptr=None, flags=0):
        Q, K, V = f32(Q), f32(K), f32(V)
        seq_lens = i32(seq_lens)
        T = int(seq_lens.sum())
        Z = np.zeros((T, d_model), dtype=np.float32)
        mask = None if mask is None else f32(mask)
        valid_lens, qk_head_ptr = i32(valid_lens), i32(qk_head_ptr)
        v_col_id, v_head_ptr = i32(v_col_id), i32(v_head_ptr)
        self.lib.orc_attention(_fp(Z), _fp(Q), _fp(K), _fp(V), Q.shape[1], V.shape[1],
                               _ipp(qk_head_ptr), _ipp(v_col_id), _ipp(v_head_ptr), _fp(mask),
                               0 if mask is None else mask.shape[1], _ipp(seq_lens),
                               _ipp(valid_lens), len(seq_lens), d_model, nhead, flags)
        return Z

    def scores(self, Q, K, d_model, nhead):
        Q, K = f32(Q), f32(K)
        L = Q.shape[0]
        S = np.zeros((nhead, L, L), dtype=np.float32)
        self.lib.orc_scores(_fp(S), _fp(Q), _fp(K), L, d_model, nhead)
        return S

    def softmax_mask(self, S, mask=None, valid=None, flags=0):
        S = f32(S).copy()
        nmat, L, _ = S.shape
        mask = None if mask is None else f32(mask)
        self.lib.orc_softmax_mask(_fp(S), _fp(mask), nmat, L, L if valid is None else valid, flags)
        return S

    def sharedqk_attention(self, S, V, d_model, nhead, mask=None, flags=0):
        S, V = f32(S), f32(V)
        L = V.shape[0]
        Z = np.zeros((L, d_model), dtype=np.float32)
        mask = None if mask is None else f32(mask)
        self.lib.orc_sharedqk_attention(_fp(Z), _fp(S), _fp(V), _fp(mask), L, d_model, nhead, flags)
        return Z

    def skip_layernorm(self, x, skip, gamma, beta):
        x = f32(x).copy()
        skip, gamma, beta = f32(skip), f32(gamma), f32(beta)
        num, size = x.shape
        self.lib.orc_skip_layernorm(_fp(x), _fp(skip), _fp(gamma), _fp(beta), num, size)
        return x

    def round_half(self, x):
        x = f32(x).copy()
        self.lib.orc_round_half(_fp(x), ctypes.c_long(x.size))
        return x

    def encoder_layer(self, X, lin, ln, seq_lens, d_model, nhead, mask=None, valid_lens=None,
                      round_half=False):
        """One post-LN encoder layer in the op order of encoder/encoder.cu:20-45.
        lin: dict name -> (row_ptr, row_offset, data, bias, N) for q,k,v,o,ffn1,ffn2.
        ln: ((gamma0, beta0), (gamma1, beta1))."""
        rh = self.round_half if round_half else (lambda a: a)
        X = f32(X)
        q = rh(self.tile_linear(X, *lin["q"][:4], lin["q"][4]))
        k = rh(self.tile_linear(X, *lin["k"][:4], lin["k"][4]))
        v = rh(self.tile_linear(X, *lin["v"][:4], lin["v"][4]))
        z = rh(self.attention(q, k, v, seq_lens, d_model, nhead, mask=mask, valid_lens=valid_lens))
        a = rh(self.tile_linear(z, *lin["o"][:4], lin["o"][4]))
        h1 = rh(self.skip_layernorm(a, X, *ln[0]))
        f = rh(self.tile_linear(h1, *lin["ffn1"][:4], lin["ffn1"][4], gelu=True))
        y = rh(self.tile_linear(f, *lin["ffn2"][:4], lin["ffn2"][4]))
        return rh(self.skip_layernorm(y, h1, *ln[1]))


_orc = None


def build_oracle():
    subprocess.run(["make", "-C", ORC_DIR, "-s"], check=True, capture_output=True)


def load():
    global _orc
    if _orc is None:
        if not os.path.exists(ORC_LIB) or os.path.getmtime(ORC_LIB) < os.path.getmtime(
                os.path.join(ORC_DIR, "et_oracle.cpp")):
            build_oracle()
        _orc = Oracle(ctypes.CDLL(ORC_LIB))
    return _orc


def load_ref():
    """ctypes handle of the reference CUDA kernels, or None if the prebuilt library is absent."""
    if not os.path.exists(REF_LIB):
        return None
    return ctypes.CDLL(REF_LIB)
