"""CPU checks of the oracle itself: fp16 conversion, generators, and every op against a plain
numpy restatement on small seeded cases."""
import numpy as np
import pytest

from tests import util


def test_half_conversion_roundtrip(orc):
    bits = np.arange(0, 1 << 16, dtype=np.uint16)
    as_f = bits.view(np.float16).astype(np.float32)
    for b in list(range(0, 1 << 16, 97)) + [0x0001, 0x03ff, 0x0400, 0x7bff, 0x7c00, 0xfbff, 0x8000]:
        f = orc.lib.orc_h2f(int(b))
        if np.isnan(as_f[b]):
            assert np.isnan(f)
            continue
        assert f == as_f[b]
        assert orc.lib.orc_f2h(f) == b
    x = util.rng(0).standard_normal(4096).astype(np.float32) * np.float32(3.0)
    x = np.concatenate([x, [65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9803e-8, 6.1e-5, -0.0]]).astype(np.float32)
    got = np.array([orc.lib.orc_f2h(float(v)) for v in x], dtype=np.uint16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert (got == want).all()


@pytest.mark.parametrize("sparsity", [0.0, 0.5, 0.9, 1.0])
def test_tile_generator_exact_count(orc, sparsity):
    nrow, ncol = 768, 3072
    rp, ro = orc.gen_sparse_tile_mat(nrow, ncol, sparsity, seed=7, bernoulli=False)
    total = (nrow // 16) * (ncol // 16)
    assert len(ro) == int(total * (1.0 - sparsity))          # test/tile_mat.cu:11
    assert rp[0] == 0 and rp[-1] == len(ro) and (np.diff(rp) >= 0).all()
    assert (ro % 16 == 0).all() and (ro >= 0).all() and (ro < ncol).all()
    for r in range(nrow // 16):                              # no duplicate tile in a block-row
        seg = ro[rp[r]:rp[r + 1]]
        assert len(np.unique(seg)) == len(seg)
    rp2, ro2 = orc.gen_sparse_tile_mat(nrow, ncol, sparsity, seed=7, bernoulli=False)
    assert (rp == rp2).all() and (ro == ro2).all()           # seeded: reproducible


def test_tile_generator_bernoulli(orc):
    rp, ro = orc.gen_sparse_tile_mat(1024, 1024, 0.8, seed=3, bernoulli=True)
    frac = len(ro) / 4096.0
    assert 0.17 < frac < 0.23
    for r in range(64):
        seg = ro[rp[r]:rp[r + 1]]
        assert (np.diff(seg) > 0).all()                      # ascending inside a block-row


def test_row_generator_and_head_ptr(orc):
    row_id = orc.gen_sparse_row_mat(768, 0.5, seed=11, nhead=12)
    assert len(row_id) == 384 and (np.diff(row_id) > 0).all()
    hp = orc.head_ptr(row_id, 12, 768)
    assert hp[0] == 0 and hp[-1] == 384
    for h in range(12):
        seg = row_id[hp[h]:hp[h + 1]]
        assert len(seg) >= 1 and (seg // 64 == h).all()
    # a head without rows is a legal input of head_ptr (repeated prefix)
    hp2 = orc.head_ptr(np.array([0, 1, 130], dtype=np.int32), 4, 256)
    assert hp2.tolist() == [0, 2, 2, 3, 3]


def test_bsr_roundtrip_bit_exact(orc):
    rp, ro, data, _ = util.make_tile_linear(orc, 128, 96, 0.6, seed=5)
    W = orc.bsr_to_dense(rp, ro, data, 96, 128)
    mask = np.zeros((6, 8), dtype=bool)
    for r in range(6):
        for i in range(rp[r], rp[r + 1]):
            mask[r, ro[i] // 16] = True
            blk = W[16 * r:16 * r + 16, ro[i]:ro[i] + 16]
            assert (blk == data[i].astype(np.float32).reshape(16, 16)).all()
    dense_mask = np.abs(W).reshape(6, 16, 8, 16).sum(axis=(1, 3)) > 0
    assert (dense_mask == mask).all()


@pytest.mark.parametrize("gelu", [False, True])
def test_tile_linear_vs_numpy(orc, gelu):
    T, K, N = 40, 128, 96
    rp, ro, data, bias = util.make_tile_linear(orc, K, N, 0.5, seed=9, bias_std=0.1)
    X = util.activations(1, (T, K))
    W = orc.bsr_to_dense(rp, ro, data, N, K).astype(np.float64)
    want = X.astype(np.float64) @ W.T + bias.astype(np.float64)
    if gelu:
        want = 0.5 * want * (1 + np.tanh(0.7978845608028654 * (want + 0.044715 * want ** 3)))
    got = orc.tile_linear(X, rp, ro, data, bias, N, gelu=gelu)
    assert np.abs(got - want).max() < 1e-4


def test_row_linear_vs_numpy(orc):
    X = util.activations(2, (33, 64))
    W = util.weights(3, (20, 64), 0.1)
    b = util.weights(4, (20,), 0.1)
    got = orc.row_linear(X, W, b, out_pitch=32)
    want = X.astype(np.float64) @ W.astype(np.float64).T + b.astype(np.float64)
    assert np.abs(got[:, :20] - want).max() < 1e-4 and (got[:, 20:] == 0).all()


def _np_attention(Q, K, V, lens, d, H, mask=None, valid=None):
    hd = d // H
    Z = np.zeros((int(np.sum(lens)), d))
    s0 = 0
    for b, L in enumerate(lens):
        vl = L if valid is None else valid[b]
        for h in range(H):
            q = Q[s0:s0 + L, h * hd:(h + 1) * hd].astype(np.float64)
            k = K[s0:s0 + vl, h * hd:(h + 1) * hd].astype(np.float64)
            v = V[s0:s0 + vl, h * hd:(h + 1) * hd].astype(np.float64)
            s = q @ k.T / np.sqrt(hd)
            if mask is not None:
                s = s + mask[:L, :vl]
            s = s - s.max(axis=1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(axis=1, keepdims=True)
            Z[s0:s0 + L, h * hd:(h + 1) * hd] = p @ v
        s0 += L
    return Z


def test_attention_vs_numpy_varlen_and_mask(orc):
    d, H = 64, 4
    lens = [5, 16, 23]
    T = sum(lens)
    Q, K, V = (util.activations(s, (T, d)) for s in (1, 2, 3))
    mask = (util.rng(4).standard_normal((32, 32)) * 0.5).astype(np.float32)
    got = orc.attention(Q, K, V, lens, d, H, mask=mask)
    want = _np_attention(Q, K, V, lens, d, H, mask=mask)
    assert np.abs(got - want).max() < 1e-5
    valid = [5, 9, 23]
    got = orc.attention(Q, K, V, lens, d, H, valid_lens=valid)
    want = _np_attention(Q, K, V, lens, d, H, valid=valid)
    assert np.abs(got - want).max() < 1e-5


def test_attention_fully_masked_row_is_zero(orc):
    d, H, L = 32, 2, 8
    Q, K, V = (util.activations(s, (L, d)) for s in (1, 2, 3))
    mask = np.zeros((L, L), dtype=np.float32)
    mask[3, :] = -np.inf
    got = orc.attention(Q, K, V, [L], d, H, mask=mask)
    assert (got[3] == 0).all() and np.isfinite(got).all()


def test_attention_pruned_scatter(orc):
    d, H, L = 64, 4, 12
    hd = d // H
    row_id = orc.gen_sparse_row_mat(d, 0.5, seed=21, nhead=H)
    hp = orc.head_ptr(row_id, H, d)
    Q, K = util.activations(1, (L, d)), util.activations(2, (L, d))
    Vc = util.activations(3, (L, len(row_id)))
    got = orc.attention(Q, K, Vc, [L], d, H, v_col_id=row_id, v_head_ptr=hp)
    Vfull = np.zeros((L, d), dtype=np.float32)
    Vfull[:, row_id] = Vc.astype(np.float32)
    want = _np_attention(Q, K, Vfull, [L], d, H)
    assert np.abs(got - want).max() < 1e-5
    dropped = np.setdiff1d(np.arange(d), row_id)
    assert (got[:, dropped] == 0).all()                      # pruned columns are exactly zero
    # Q/K compact with shared retained dims
    Qc, Kc = Q[:, row_id], K[:, row_id]
    got2 = orc.attention(Qc, Kc, Vc, [L], d, H, qk_head_ptr=hp, v_col_id=row_id, v_head_ptr=hp)
    Qz, Kz = np.zeros((L, d), np.float32), np.zeros((L, d), np.float32)
    Qz[:, row_id], Kz[:, row_id] = Qc, Kc
    want2 = _np_attention(Qz, Kz, Vfull, [L], d, H)
    assert np.abs(got2 - want2).max() < 1e-5
    assert hd == 16


def test_scores_softmax_sharedqk_consistent(orc):
    d, H, L = 64, 4, 16
    Q, K, V = (util.activations(s, (L, d)) for s in (1, 2, 3))
    mask = (util.rng(4).standard_normal((L, L)) * 0.5).astype(np.float32)
    S = orc.scores(Q, K, d, H)
    Z1 = orc.sharedqk_attention(S, V, d, H, mask=mask)
    Z2 = orc.attention(Q, K, V, [L], d, H, mask=mask)
    assert np.abs(Z1 - Z2).max() < 1e-5
    P = orc.softmax_mask(S, mask)
    assert np.abs(P.sum(axis=2) - 1).max() < 1e-5
    P2 = orc.softmax_mask(S, mask, valid=10)
    assert (P2[:, :, 10:] == 0).all() and np.abs(P2.sum(axis=2) - 1).max() < 1e-5


def test_ref_compat_softmax_is_base2_with_zero_floor(orc):
    S = np.array([[[-1.0, -2.0, -3.0, -0.5]]], dtype=np.float32).repeat(4, axis=1)
    P = orc.softmax_mask(S, flags=1)
    e = np.exp2(S[0, 0] - 0.0)                              # max floor at 0, base 2
    assert np.abs(P[0, 0] - e / e.sum()).max() < 1e-6


def test_skip_layernorm_vs_numpy(orc):
    x, s = util.activations(1, (9, 768)), util.activations(2, (9, 768))
    g, b = util.weights(3, (768,), 1.0), util.weights(4, (768,), 1.0)
    got = orc.skip_layernorm(x, s, g, b)
    v = x.astype(np.float64) + s.astype(np.float64)
    mu = v.mean(axis=1, keepdims=True)
    var = ((v - mu) ** 2).mean(axis=1, keepdims=True)
    want = (v - mu) / np.sqrt(var + 1e-6) * g.astype(np.float64) + b.astype(np.float64)
    assert np.abs(got - want).max() < 1e-4
