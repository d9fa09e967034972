"""GPU parity tests of the attention family and the row-pruned linear against the CPU oracle."""
import ctypes

import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.float().cpu().numpy()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def et():
    import et_b200
    et_b200.lib()
    return et_b200


def _qkv(seed, T, d, std=1.0):
    return [(util.activations(seed + i, (T, d)).astype(np.float32) * std).astype(np.float16) for i in range(3)]


@pytest.mark.parametrize("L,d,H,use_mask", [(128, 768, 12, False), (128, 768, 12, True), (256, 768, 12, True),
                                            (512, 1024, 16, False), (16, 128, 2, True), (77, 768, 12, True),
                                            (1, 64, 1, False), (200, 256, 8, False), (2048, 128, 2, False),
                                            (1100, 128, 2, True)])
def test_attention_otf(et, orc, L, d, H, use_mask):
    Q, K, V = _qkv(1, L, d)
    mask = None
    if use_mask:
        mask = (util.rng(9).standard_normal((L, L)) * 0.5).astype(np.float16)
        mask[:, L // 3] = -10000.0
    want = orc.attention(Q, K, V, [L], d, H, mask=mask)
    out = torch.full((L, d), float("nan"), dtype=torch.float16, device="cuda")
    et.attention_otf(out, dev(Q), dev(K), dev(V), None if mask is None else dev(mask), L, d, H)
    torch.cuda.synchronize()
    util.assert_close(host(out), want, what=f"otf attention L={L}")


@pytest.mark.parametrize("scale,fp32_scores,max_abs,mean_abs", [(1.0, False, 4e-3, 2e-4), (1.0, True, 4e-3, 2e-4),
                                                                  (3.0, True, 6e-3, 4e-4), (3.0, False, 6e-2, 3e-3)])
def test_attention_score_precision(et, orc, scale, fp32_scores, max_abs, mean_abs):
    """Q K^T accumulated in fp16 (the default, as the reference does) or in fp32: with unit-variance operands
    (|q.k| up to ~45) both stay within a fifth of the parity tolerance; with operands three times larger (|q.k| up to
    ~390, softmax close to one-hot) the fp32 form still does and the fp16 form is allowed the error of rounding the
    scores to fp16."""
    L, d, H = 512, 768, 12
    Q, K, V = _qkv(1, L, d)
    Q = (Q.astype(np.float32) * scale).astype(np.float16)
    K = (K.astype(np.float32) * scale).astype(np.float16)
    want = orc.attention(Q, K, V, [L], d, H)
    assert not et.attention_scores_fp32()
    et.set_attention_scores_fp32(fp32_scores)
    try:
        assert et.attention_scores_fp32() == fp32_scores
        out = torch.full((L, d), float("nan"), dtype=torch.float16, device="cuda")
        et.attention_otf(out, dev(Q), dev(K), dev(V), None, L, d, H)
        torch.cuda.synchronize()
    finally:
        et.set_attention_scores_fp32(False)
    util.assert_close(host(out), want, max_abs=max_abs, mean_abs=mean_abs, what=f"scores fp32={fp32_scores}, scale {scale}")


def test_attention_otf_matches_reference_kernel_in_base2_mode(et, orc, ref):
    """The shipped kernel exponentiates in base 2 and floors the row max at 0; with its scale multiplied by
    log2(e) and scores that stay positive-max it computes a true softmax, comparable with ours."""
    L, d, H = 128, 768, 12
    Q, K, V = _qkv(3, L, d, std=0.5)
    mask = np.zeros((L, L), dtype=np.float16)
    Qd, Kd, Vd, Md = dev(Q), dev(K), dev(V), dev(mask)
    outr = torch.zeros((L, d), dtype=torch.float16, device="cuda")
    scale = float(1.4426950408889634 / np.sqrt(d // H))
    rc = ref.ref_otf_attention(_p(outr), _p(Qd), _p(Kd), _p(Vd), _p(Md), L, d, H, ctypes.c_float(scale), None)
    torch.cuda.synchronize()
    assert rc == 0
    want = orc.attention(Q, K, V, [L], d, H)
    util.assert_close(host(outr), want, max_abs=6e-2, mean_abs=6e-3, what="reference OTF vs oracle")
    out = torch.zeros((L, d), dtype=torch.float16, device="cuda")
    et.attention_otf(out, Qd, Kd, Vd, Md, L, d, H)
    torch.cuda.synchronize()
    util.assert_close(host(out), host(outr), max_abs=6e-2, mean_abs=6e-3, what="new vs reference OTF")
    # as shipped (scale without log2 e): the oracle's compatibility mode reproduces it
    rc = ref.ref_otf_attention(_p(outr), _p(Qd), _p(Kd), _p(Vd), _p(Md), L, d, H, ctypes.c_float(-1.0), None)
    torch.cuda.synchronize()
    assert rc == 0
    from tests.oracle_lib import REF_COMPAT
    want2 = orc.attention(Q, K, V, [L], d, H, flags=REF_COMPAT)
    util.assert_close(host(outr), want2, max_abs=6e-2, mean_abs=6e-3, what="reference OTF as shipped vs compat oracle")


def test_attention_fully_masked_row_and_zero_valid(et, orc):
    L, d, H = 64, 128, 2
    Q, K, V = _qkv(5, L, d)
    mask = np.zeros((L, L), dtype=np.float16)
    mask[7, :] = -np.inf
    out = torch.full((L, d), float("nan"), dtype=torch.float16, device="cuda")
    et.attention_otf(out, dev(Q), dev(K), dev(V), dev(mask), L, d, H)
    torch.cuda.synchronize()
    got = host(out)
    assert np.isfinite(got).all() and (got[7] == 0).all()
    util.assert_close(got, orc.attention(Q, K, V, [L], d, H, mask=mask.astype(np.float32)), what="masked row")


@pytest.mark.parametrize("lens", [[5, 16, 23, 64, 65, 130], [512, 32, 33, 100], [1], [0, 7, 0, 128]])
def test_attention_batch_varlen(et, orc, lens):
    d, H = 768, 12
    T = sum(lens)
    Q, K, V = _qkv(11, max(T, 1), d)
    Q, K, V = Q[:T], K[:T], V[:T]
    want = orc.attention(Q, K, V, lens, d, H)
    cu = dev(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32))
    out = torch.full((T, d), float("nan"), dtype=torch.float16, device="cuda")
    et.attention_batch(out, dev(Q), dev(K), dev(V), d, H, cu_seqlens=cu, batch=len(lens), total_tokens=T,
                       max_seq_len=max(lens))          # tensor-core kernel (all lengths <= 512)
    torch.cuda.synchronize()
    util.assert_close(host(out), want, what=f"varlen attention {lens}")
    out2 = torch.full((T, d), float("nan"), dtype=torch.float16, device="cuda")
    et.attention_batch(out2, dev(Q), dev(K), dev(V), d, H, cu_seqlens=cu, batch=len(lens), total_tokens=T)
    torch.cuda.synchronize()                           # longest length not given: general kernel
    util.assert_close(host(out2), want, what=f"varlen attention, general kernel {lens}")


def test_attention_batch_key_padding_equals_unpadded(et, orc):
    """Padded layout with valid_lens gives, on the valid rows, exactly the unpadded result."""
    d, H, S = 256, 4, 96
    lens = [40, 96, 17, 64]
    B = len(lens)
    Q, K, V = _qkv(21, B * S, d)
    valid = dev(np.array(lens, dtype=np.int32))
    out_pad = torch.zeros((B * S, d), dtype=torch.float16, device="cuda")
    et.attention_batch(out_pad, dev(Q), dev(K), dev(V), d, H, valid_lens=valid, batch=B, uniform_len=S)
    rows = np.concatenate([np.arange(b * S, b * S + lens[b]) for b in range(B)])
    cu = dev(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32))
    out_var = torch.zeros((len(rows), d), dtype=torch.float16, device="cuda")
    et.attention_batch(out_var, dev(Q[rows]), dev(K[rows]), dev(V[rows]), d, H, cu_seqlens=cu, batch=B,
                       max_seq_len=max(lens))
    torch.cuda.synchronize()
    assert torch.equal(out_pad[torch.from_numpy(rows).cuda()], out_var)
    want = orc.attention(Q, K, V, [S] * B, d, H, valid_lens=lens)
    util.assert_close(host(out_pad), want, what="key-padded attention")


def test_attention_prune_scatter(et, orc):
    L, d, H = 256, 768, 12
    row_id = orc.gen_sparse_row_mat(d, 0.5, seed=5, nhead=H)
    hp = orc.head_ptr(row_id, H, d)
    nnz = len(row_id)
    Q, K = util.activations(1, (L, d)), util.activations(2, (L, d))
    Vc = util.activations(3, (L, nnz))
    want = orc.attention(Q, K, Vc, [L], d, H, v_col_id=row_id, v_head_ptr=hp)
    out = torch.full((L, d), float("nan"), dtype=torch.float16, device="cuda")
    et.attention_prune(out, dev(Q), dev(K), dev(Vc), dev(row_id), dev(hp), nnz, None, L, d, H)
    torch.cuda.synchronize()
    got = host(out)
    util.assert_close(got, want, what="pruned-V attention")
    dropped = np.setdiff1d(np.arange(d), row_id)
    assert (got[:, dropped] == 0).all()          # pruned columns are exactly zero


def test_attention_qk_and_v_pruned(et, orc):
    L, d, H = 100, 768, 12
    row_id = orc.gen_sparse_row_mat(d, 0.5, seed=6, nhead=H)
    hp = orc.head_ptr(row_id, H, d)
    nnz = len(row_id)
    Qc, Kc, Vc = (util.activations(s, (L, nnz)) for s in (1, 2, 3))
    want = orc.attention(Qc, Kc, Vc, [L], d, H, qk_head_ptr=hp, v_col_id=row_id, v_head_ptr=hp)
    out = torch.full((L, d), float("nan"), dtype=torch.float16, device="cuda")
    hpd, rid = dev(hp), dev(row_id)
    et.attention_batch(out, dev(Qc), dev(Kc), dev(Vc), d, H, batch=1, uniform_len=L, qk_head_ptr=hpd,
                       v_col_id=rid, v_head_ptr=hpd)
    torch.cuda.synchronize()
    util.assert_close(host(out), want, what="Q/K/V-pruned attention")


@pytest.mark.parametrize("L", [128, 72])
def test_scores_then_sharedqk(et, orc, L):
    d, H = 768, 12
    Q, K, V = _qkv(31, L, d)
    mask = (util.rng(9).standard_normal((L, L)) * 0.5).astype(np.float16)
    S = torch.zeros((H, L, L), dtype=torch.float16, device="cuda")
    et.qk_scores(S, dev(Q), dev(K), L, d, H)
    torch.cuda.synchronize()
    util.assert_close(host(S), orc.scores(Q, K, d, H), what="qk scores")
    out = torch.zeros((L, d), dtype=torch.float16, device="cuda")
    et.attention_sharedqk(out, S, dev(V), dev(mask), L, d, H)
    torch.cuda.synchronize()
    want = orc.sharedqk_attention(host(S), V, d, H, mask=mask)
    util.assert_close(host(out), want, what="sharedQK attention")
    util.assert_close(host(out), orc.attention(Q, K, V, [L], d, H, mask=mask), what="sharedQK vs on-the-fly")


def test_sharedqk_matches_reference_kernel_with_zero_mask(et, orc, ref):
    L, d, H = 128, 768, 12
    Q, K, V = _qkv(41, L, d, std=0.5)
    S = (orc.scores(Q, K, d, H) * 1.4426950408889634).astype(np.float16)   # base-2 kernel: pre-scale by log2 e
    Sd, Vd, Md = dev(S), dev(V), torch.zeros((L, L), dtype=torch.float16, device="cuda")
    outr = torch.zeros((L, d), dtype=torch.float16, device="cuda")
    rc = ref.ref_sharedqk_attention(_p(outr), _p(Sd), _p(Vd), _p(Md), L, d, H)
    torch.cuda.synchronize()
    assert rc == 0
    want = orc.attention(Q, K, V, [L], d, H)
    util.assert_close(host(outr), want, max_abs=6e-2, mean_abs=6e-3, what="reference sharedQK vs oracle")


def test_row_linear_and_meta(et, orc):
    T, K, N, H = 300, 768, 768, 12
    row_id = orc.gen_sparse_row_mat(N, 0.5, seed=8, nhead=H)
    W = util.weights(1, (len(row_id), K))
    b = util.weights(2, (len(row_id),), 0.1)
    X = util.activations(3, (T, K))
    w = et.RowWeight(K, N, T, W, row_id, b, H)
    assert w.row_id_size == len(row_id) and w.nrow == (len(row_id) + 15) // 16 * 16
    assert (w.head_ptr == orc.head_ptr(row_id, H, N)).all()                 # bit-exact index structure
    out = torch.full((T, w.nrow), float("nan"), dtype=torch.float16, device="cuda")
    w.run(out, dev(X))
    torch.cuda.synchronize()
    want = orc.row_linear(X, W, b, out_pitch=w.nrow)
    util.assert_close(host(out), want, what="row-pruned linear")
    # ragged keep count (not a multiple of 16): padding columns are exactly zero
    row_id2 = row_id[:-5]
    w2 = et.RowWeight(K, N, T, W[:-5], row_id2, b[:-5], H)
    out2 = torch.full((T, w2.nrow), float("nan"), dtype=torch.float16, device="cuda")
    w2.run(out2, dev(X))
    torch.cuda.synchronize()
    got2 = host(out2)
    util.assert_close(got2, orc.row_linear(X, W[:-5], b[:-5], out_pitch=w2.nrow), what="row-pruned ragged")
    assert (got2[:, len(row_id2):] == 0).all()


def test_row_linear_matches_reference_cublas_path(et, orc, ref):
    T, K, N, H = 256, 768, 768, 12
    row_id = orc.gen_sparse_row_mat(N, 0.5, seed=8, nhead=H)     # 384 rows: a multiple of 16
    W = util.weights(1, (len(row_id), K))
    b = util.weights(2, (len(row_id),), 0.1)
    X = util.activations(3, (T, K))
    Xd, Wd, bd = dev(X), dev(W), dev(b)
    outr = torch.zeros((T, len(row_id)), dtype=torch.float16, device="cuda")
    rc = ref.ref_row_spmm(_p(outr), _p(Xd), _p(Wd), _p(bd), T, len(row_id), K, None)
    torch.cuda.synchronize()
    assert rc == 0
    w = et.RowWeight(K, N, T, W, row_id, b, H)
    out = torch.zeros((T, w.nrow), dtype=torch.float16, device="cuda")
    w.run(out, Xd)
    torch.cuda.synchronize()
    util.assert_close(host(out), host(outr), what="row-pruned linear vs reference cuBLAS path")


def test_generators_bit_exact_with_oracle(et, orc):
    for (nrow, ncol, s, seed, bern) in [(768, 768, 0.5, 1, False), (3072, 768, 0.9, 2, False),
                                        (768, 3072, 0.75, 3, True), (1024, 4096, 0.8, 4, True),
                                        (64, 64, 0.0, 5, False), (64, 64, 1.0, 6, True)]:
        rp, ro = et.gen_sparse_tile_mat(nrow, ncol, s, seed, bern)
        rp2, ro2 = orc.gen_sparse_tile_mat(nrow, ncol, s, seed, bern)
        assert (rp == rp2).all() and (ro == ro2).all()
    for (nrow, s, seed, H) in [(768, 0.5, 1, 12), (1024, 0.75, 2, 16), (768, 0.9, 3, 12)]:
        a, b = et.gen_sparse_row_mat(nrow, s, seed, H), orc.gen_sparse_row_mat(nrow, s, seed, H)
        assert (a == b).all()
        assert (et.build_head_ptr(a, H, nrow) == orc.head_ptr(b, H, nrow)).all()
