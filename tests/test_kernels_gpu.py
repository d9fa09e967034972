"""GPU parity tests: every CUDA entry point of the C-ABI library against the CPU oracle on the same
seeded inputs (fp16 result vs fp32 oracle: max-abs <= 2e-2, mean-abs <= 2e-3), plus the reference
project's own CUDA kernels where they are usable as shipped."""
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


# ------------------------------------------------------------------ skip LayerNorm
@pytest.mark.parametrize("num,size", [(1, 768), (7, 768), (2048, 768), (515, 1024), (33, 256),
                                      (5, 2048), (9, 200), (3, 1538)])
def test_skip_layernorm(et, orc, num, size):
    x, s = util.activations(1, (num, size)), util.activations(2, (num, size))
    g = (1.0 + util.weights(3, (size,), 0.2).astype(np.float32)).astype(np.float16)
    b = util.weights(4, (size,), 0.2)
    want = orc.skip_layernorm(x, s, g, b)
    xd = dev(x)
    et.skip_layernorm(xd, dev(s), dev(g), dev(b))
    torch.cuda.synchronize()
    util.assert_close(host(xd), want, what=f"skip_layernorm {num}x{size}")


def test_skip_layernorm_matches_reference_kernels(et, orc, ref):
    for num, size in [(128, 768), (2048, 768), (1024, 1024)]:   # v1 and v2 kernels of the reference
        x, s = util.activations(1, (num, size)), util.activations(2, (num, size))
        g = (1.0 + util.weights(3, (size,), 0.2).astype(np.float32)).astype(np.float16)
        b = util.weights(4, (size,), 0.2)
        want = orc.skip_layernorm(x, s, g, b)
        xr, sd, gd, bd = dev(x), dev(s), dev(g), dev(b)   # keep the tensors alive across the launch
        rc = ref.ref_skip_layernorm(_p(xr), _p(sd), _p(gd), _p(bd), num, size, None)
        torch.cuda.synchronize()
        assert rc == 0
        # the reference adds, centres and scales in fp16 in its second kernel: looser bound
        util.assert_close(host(xr), want, max_abs=6e-2, mean_abs=6e-3, what="reference LN vs oracle")
        xd = dev(x)
        et.skip_layernorm(xd, sd, gd, bd)
        torch.cuda.synchronize()
        util.assert_close(host(xd), host(xr), max_abs=6e-2, mean_abs=6e-3, what="new vs reference LN")


def test_skip_layernorm_bad_args(et):
    x = torch.zeros(4, 768, dtype=torch.float16, device="cuda")
    with pytest.raises(et.EtError):
        et.check(et.lib().et_skip_layernorm(None, _p(x), _p(x), _p(x), 4, 768, None))
    with pytest.raises(et.EtError):
        et.check(et.lib().et_skip_layernorm(_p(x), _p(x), _p(x), _p(x), 4, 0, None))
    et.check(et.lib().et_skip_layernorm(_p(x), _p(x), _p(x), _p(x), 0, 768, None))  # empty is fine


# ------------------------------------------------------------------ mask + softmax
@pytest.mark.parametrize("nmat,L,valid,use_mask", [(12, 128, None, True), (3, 256, 200, True),
                                                   (2, 512, None, False), (5, 40, 33, True),
                                                   (2, 77, None, True), (1, 1024, 1000, False)])
def test_softmax_mask(et, orc, nmat, L, valid, use_mask):
    S = (util.rng(5).standard_normal((nmat, L, L)) * 3).astype(np.float16)
    mask = (util.rng(6).standard_normal((L, L))).astype(np.float16) if use_mask else None
    if use_mask:
        mask[:, L // 2] = -10000.0          # a padded key column
    want = orc.softmax_mask(S, mask, valid)
    Sd = dev(S)
    et.softmax_mask(Sd, None if mask is None else dev(mask), valid)
    torch.cuda.synchronize()
    got = host(Sd)
    util.assert_close(got, want, what=f"softmax {nmat}x{L}")
    if valid is not None:
        assert (got[:, :, valid:] == 0).all()


def test_softmax_fully_masked_row_is_zero(et):
    L = 64
    S = dev(util.activations(1, (2, L, L)))
    et.softmax_mask(S, None, 0)
    torch.cuda.synchronize()
    assert (host(S) == 0).all()


# ------------------------------------------------------------------ tile-pruned linear
def _run_tile(et, orc, T, K, N, sparsity, seed, gelu=False, bernoulli=True, bias_std=0.05, size=None):
    rp, ro, data, bias = util.make_tile_linear(orc, K, N, sparsity, seed, bernoulli, bias_std)
    X = util.activations(seed + 10, (T, K))
    want = orc.tile_linear(X, rp, ro, data, bias, N, gelu=gelu)
    w = et.TileWeight(K, N, T if size is None else size, data, rp, ro, bias, is_gelu=gelu)
    Y = torch.full((T, N), float("nan"), dtype=torch.float16, device="cuda")
    w.run(Y, dev(X))
    torch.cuda.synchronize()
    w.check()
    return host(Y), want, w


@pytest.mark.parametrize("T,K,N,sparsity,gelu", [
    (128, 64, 16, 0.0, False),        # one tile column, one block-row
    (128, 768, 768, 0.5, False),
    (2048, 768, 768, 0.75, False),
    (2048, 768, 3072, 0.5, True),
    (2048, 3072, 768, 0.9, False),
    (300, 768, 768, 0.0, False),      # dense, ragged token count
    (1, 256, 48, 0.5, True),
    (4096, 1024, 1024, 0.8, False),
    (200, 80, 112, 0.3, False),       # K not a multiple of 64, N not a multiple of the chunk
])
def test_tile_linear(et, orc, T, K, N, sparsity, gelu):
    got, want, _ = _run_tile(et, orc, T, K, N, sparsity, seed=T + K + N, gelu=gelu)
    util.assert_close(got, want, what=f"tile linear T={T} K={K} N={N} s={sparsity}")


def test_tile_linear_exact_count_shuffled_order_and_empty_rows(et, orc):
    # exact-count generator lists a block-row's tiles in shuffle order; at 95 % many block-rows are empty
    got, want, _ = _run_tile(et, orc, 256, 768, 768, 0.95, seed=77, bernoulli=False)
    util.assert_close(got, want, what="tile linear exact-count")
    got, want, _ = _run_tile(et, orc, 256, 768, 768, 1.0, seed=78, bernoulli=False, bias_std=0.3)
    util.assert_close(got, want, what="tile linear all tiles pruned (bias only)")


@pytest.mark.parametrize("size_hint", [128, 2048, 131072])
def test_tile_linear_all_chunkings(et, orc, size_hint):
    got, want, w = _run_tile(et, orc, 384, 768, 3072, 0.75, seed=3, gelu=True, size=size_hint)
    util.assert_close(got, want, what=f"tile linear hint {size_hint} {w.info()}")


@pytest.mark.parametrize("T,K,N,sparsity,gelu", [
    (2048, 768, 2304, 0.75, False),   # the fused Q|K|V shape of the 16 x 128 tile layer
    (2048, 768, 768, 0.75, False),
    (2048, 768, 3072, 0.75, True),
    (2048, 3072, 768, 0.75, False),
    (2048, 768, 768, 0.5, False),
    (4096, 1024, 4096, 0.8, True),    # BERT-large FFN1 slab count above one wave of two-tile CTAs
    (300, 768, 3072, 0.9, True),      # ragged token count, under-filled grid, odd tile count per CTA
])
def test_tile_linear_packed_for_throughput(et, orc, T, K, N, sparsity, gelu):
    """Weights packed under the throughput goal (larger chunks, two tiles per CTA): the configuration a caller
    with several batches in flight uses. Same oracle, same tolerance."""
    et.set_tuning_goal("throughput")
    try:
        got, want, w = _run_tile(et, orc, T, K, N, sparsity, seed=T + K + N + 1, gelu=gelu)
    finally:
        et.set_tuning_goal("latency")
    util.assert_close(got, want, what=f"tile linear (throughput packing) T={T} K={K} N={N} s={sparsity} {w.info()}")


def test_tile_linear_pruned_tiles_do_not_contribute(et, orc):
    """Mask exactness: output equals the dense product with the pruned tiles zeroed, and does not
    change when garbage is placed where the pruned tiles would be."""
    T, K, N = 128, 256, 64
    rp, ro, data, bias = util.make_tile_linear(orc, K, N, 0.5, seed=4)
    W = orc.bsr_to_dense(rp, ro, data, N, K)
    X = util.activations(5, (T, K))
    w = et.TileWeight(K, N, T, data, rp, ro, bias)
    Y = torch.zeros((T, N), dtype=torch.float16, device="cuda")
    w.run(Y, dev(X))
    torch.cuda.synchronize()
    w.check()
    want = X.astype(np.float32) @ W.T
    util.assert_close(host(Y), want, what="tile linear vs masked dense")


def test_tile_linear_matches_reference_kernel(et, orc, ref):
    T, K, N = 768, 768, 768
    for gelu in (0, 1):
        rp, ro, data, bias = util.make_tile_linear(orc, K, N, 0.5, seed=31, bias_std=0.05)
        X = util.activations(32, (T, K))
        want = orc.tile_linear(X, rp, ro, data, bias, N, gelu=bool(gelu))
        Yr = torch.zeros((T, N), dtype=torch.float16, device="cuda")
        Xd, rpd, rod, dd, bd = dev(X), dev(rp), dev(ro), dev(data), dev(bias)
        rc = ref.ref_tile_spmm(_p(Yr), _p(Xd), _p(rpd), _p(rod), _p(dd), T, N, K, _p(bd), gelu, None)
        torch.cuda.synchronize()
        assert rc == 0
        util.assert_close(host(Yr), want, max_abs=4e-2, mean_abs=4e-3, what="reference tile GEMM vs oracle")
        w = et.TileWeight(K, N, T, data, rp, ro, bias)
        Y = torch.zeros((T, N), dtype=torch.float16, device="cuda")
        w.run(Y, Xd, gelu=bool(gelu))
        torch.cuda.synchronize()
        util.assert_close(host(Y), host(Yr), max_abs=4e-2, mean_abs=4e-3, what="new vs reference tile GEMM")


def test_tile_spmm_raw_launcher(et, orc):
    T, K, N = 256, 768, 768
    rp, ro, data, bias = util.make_tile_linear(orc, K, N, 0.75, seed=41, bias_std=0.05)
    X = util.activations(42, (T, K))
    want = orc.tile_linear(X, rp, ro, data, bias, N)
    Y = torch.zeros((T, N), dtype=torch.float16, device="cuda")
    drp, dro, dd, db = dev(rp), dev(ro), dev(data), dev(bias)
    for _ in range(2):   # second call hits the packed-weight cache
        et.tile_spmm_bias(Y, dev(X), drp, dro, dd, db, K=K)
        torch.cuda.synchronize()
        util.assert_close(host(Y), want, what="raw tile launcher")
    et.tile_spmm_cache_clear()


def test_tile_weight_rejects_malformed_format(et):
    data = np.zeros((2, 256), dtype=np.float16)
    ok_rp = np.array([0, 1, 2], dtype=np.int32)
    with pytest.raises(et.EtError):   # offset not a multiple of 16
        et.TileWeight(64, 32, 128, data, ok_rp, np.array([8, 16], dtype=np.int32))
    with pytest.raises(et.EtError):   # offset beyond in_feat
        et.TileWeight(64, 32, 128, data, ok_rp, np.array([0, 64], dtype=np.int32))
    with pytest.raises(et.EtError):   # row_ptr does not end at ntile
        et.TileWeight(64, 32, 128, data, np.array([0, 1, 1], dtype=np.int32), np.array([0, 16], dtype=np.int32))
    with pytest.raises(et.EtError):   # not monotone
        et.TileWeight(64, 48, 128, data, np.array([0, 2, 1, 2], dtype=np.int32), np.array([0, 16], dtype=np.int32))
    with pytest.raises(et.EtError):   # features not multiples of 16
        et.TileWeight(60, 32, 128, data, ok_rp, np.array([0, 16], dtype=np.int32))
