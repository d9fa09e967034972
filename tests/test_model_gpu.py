"""GPU tests of the layer stack (et_model_*) and of ingested real weights: a stack equals its layers run one by
one (bit-exact) and the oracle's layers chained (tolerance); magnitude-pruned weights give the masked-dense result."""
import numpy as np
import pytest

from tests import util
from tests.test_encoder_gpu import build_encoder, dev, host, make_layer, orc_lin

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def et():
    import et_b200
    et_b200.lib()
    return et_b200


def test_model_equals_layers_one_by_one_and_oracle(et, orc):
    d, H, dff, n_layers = 256, 4, 1024, 3
    lens = [50, 128, 17, 96]
    T = sum(lens)
    layers = [make_layer(orc, d, dff, 0.5, seed=20 + 7 * i) for i in range(n_layers)]
    X = util.activations(31, (T, d))
    # oracle: layers chained in fp32 with fp16 storage between layers (what the GPU path stores)
    want = X
    for lin, ln in layers:
        want = orc.encoder_layer(np.asarray(want, dtype=np.float16), orc_lin(lin), ln, lens, d, H).astype(np.float16)
    # layers one by one through the single-layer object
    singles = [build_encoder(et, et.KIND_TILE, lin, ln, d, 128, H, T) for lin, ln in layers]
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, d, T, len(lens), 128, H) // 2,
                          dtype=torch.float16, device="cuda")
    x = dev(X)
    step = torch.zeros_like(x)
    cur = x
    for enc in singles:
        enc.run_batch(step, cur, lens, scratch)
        cur = step.clone()
    torch.cuda.synchronize()
    # the stack with separate LayerNorms: direct run, captured run, replayed run must all agree bit for bit with the chain
    model = et.Model([build_encoder(et, et.KIND_TILE, lin, ln, d, 128, H, T) for lin, ln in layers])
    assert model.num_layers == n_layers and not model.layernorm_fused
    out = torch.zeros_like(x)
    for call in range(4):
        out.zero_()
        model.run_batch(out, x, lens)
        torch.cuda.synchronize()
        assert torch.equal(out, cur), f"call {call}"
    util.assert_close(host(out), want.astype(np.float32), max_abs=4e-2, mean_abs=4e-3, what="3-layer stack vs oracle")
    # the optional form, LayerNorms folded into the linears: same oracle, same tolerance, calls identical to each other
    model.set_layernorm_fusion(True)
    assert model.layernorm_fused
    first = None
    for call in range(4):
        out.fill_(float("nan"))
        model.run_batch(out, x, lens)
        torch.cuda.synchronize()
        util.assert_close(host(out), want.astype(np.float32), max_abs=4e-2, mean_abs=4e-3, what=f"3-layer stack, folded LayerNorms, call {call}")
        first = out.clone() if first is None else first
        assert torch.equal(out, first), f"folded LayerNorms, call {call}"
    model.check()
    model.set_layernorm_fusion(False)
    # in place, equal lengths, no graphs
    model.set_graph_replay(False)
    xe = dev(util.activations(32, (3 * 64, d)))
    ref = torch.zeros_like(xe)
    model.run_batch(ref, xe, [64] * 3)
    model.run_batch(xe, xe, [64] * 3)
    torch.cuda.synchronize()
    assert torch.equal(xe, ref)


@pytest.mark.parametrize("kind_name", ["tile", "length"])
def test_model_folded_layernorms_with_unit_scale_weights(et, orc, kind_name):
    """Three layers with weights scaled so that every branch is as large as the residual, LayerNorm gamma and beta away
    from 1 and 0, ragged lengths: the folded form (gamma multiplied into the next linear's weights, mean and 1/std
    applied in its epilogue, the residual recomputed from the un-normalised tensor) against the oracle's chain, and
    against the same stack with separate LayerNorms."""
    d, H, dff, n_layers = 256, 4, 1024, 3
    lens = [128, 37, 90, 5]
    T = sum(lens)
    kind = et.KIND_TILE if kind_name == "tile" else et.KIND_LENGTH
    layers = [make_layer(orc, d, dff, 0.5, seed=90 + 7 * i, unit_scale=True) for i in range(n_layers)]
    X = util.activations(91, (T, d))
    want = X
    for lin, ln in layers:
        want = orc.encoder_layer(np.asarray(want, dtype=np.float16), orc_lin(lin), ln, lens, d, H).astype(np.float16)
    x = dev(X)
    model = et.Model([build_encoder(et, kind, lin, ln, d, 128, H, T) for lin, ln in layers])
    model.set_layernorm_fusion(True)
    assert model.layernorm_fused
    out = torch.zeros_like(x)
    for call in range(3):
        out.fill_(float("nan"))
        model.run_batch(out, x, lens)
        torch.cuda.synchronize()
        util.assert_close(host(out), want.astype(np.float32), max_abs=6e-2, mean_abs=6e-3, what=f"folded LayerNorms, unit scale, call {call}")
    model.check()
    plain = torch.zeros_like(x)
    model.set_layernorm_fusion(False)
    model.run_batch(plain, x, lens)
    torch.cuda.synchronize()
    util.assert_close(host(plain), want.astype(np.float32), max_abs=6e-2, mean_abs=6e-3, what="separate LayerNorms, unit scale")
    util.assert_close(host(out), host(plain), max_abs=4e-2, mean_abs=4e-3, what="folded against separate LayerNorms")
    # in place (out aliases in)
    model.set_layernorm_fusion(True)
    xi = x.clone()
    model.run_batch(xi, xi, lens)
    torch.cuda.synchronize()
    assert torch.equal(xi, out)


def test_model_alternating_batch_sizes(et, orc):
    """The stack's own array of lengths grows when a larger batch arrives; graphs recorded before that are
    re-recorded, and every call matches a run without graph replay."""
    d, H, dff, n_layers = 256, 4, 1024, 2
    layers = [make_layer(orc, d, dff, 0.5, seed=60 + 7 * i) for i in range(n_layers)]
    model = et.Model([build_encoder(et, et.KIND_TILE, lin, ln, d, 128, H, 512) for lin, ln in layers])
    plain = et.Model([build_encoder(et, et.KIND_TILE, lin, ln, d, 128, H, 512) for lin, ln in layers])
    plain.set_graph_replay(False)
    cases = {"a": [50, 128, 17, 96], "b": [64, 33, 128, 90, 5, 77, 128, 100], "c": [8 + (5 * i) % 40 for i in range(70)]}
    data = {}
    for name, lens in cases.items():
        x = dev(util.activations(70 + len(lens), (sum(lens), d)))
        want = torch.zeros_like(x)
        plain.run_batch(want, x, lens)
        data[name] = (lens, x, torch.zeros_like(x), want)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    for name in ("a", "a", "a", "b", "b", "b", "a", "a", "c", "c", "c", "a", "b"):
        lens, x, out, want = data[name]
        out.fill_(float("nan"))
        with torch.cuda.stream(stream):
            model.run_batch(out, x, lens)
        torch.cuda.synchronize()
        assert torch.equal(out, want), f"case {name}"
    model.check()


def test_model_repeated_ragged_calls_are_identical_and_clean(et, orc):
    """Twelve BERT-base layers on 64 sequences of length U[32,512], packed and padded, many calls: every call equals
    the first bit for bit and no bounded device-side wait gives up. (Three-stage rings at these shapes: a mover warp
    once read a stale barrier parity there when a later chunk's copy landed before an earlier one's, a race that
    shows only as an occasional wrong or abandoned launch.)"""
    d, H, dff, S, B = 768, 12, 3072, 512, 64
    lens = np.random.default_rng(4242).integers(32, S + 1, size=B).tolist()
    lin, ln = make_layer(orc, d, dff, 0.75, seed=77)
    model = et.Model([build_encoder(et, et.KIND_LENGTH, lin, ln, d, S, H, B * S) for _ in range(12)])
    stream = torch.cuda.Stream()
    xp = dev(util.activations(78, (sum(lens), d)))
    xf = dev(util.activations(79, (B * S, d)))
    yp, yf = torch.zeros_like(xp), torch.zeros_like(xf)
    # rows past a sequence's valid length are not defined in the padded form: compare the valid ones
    valid = torch.zeros(B * S, dtype=torch.bool, device="cuda")
    for b, n in enumerate(lens):
        valid[b * S: b * S + n] = True
    cases = (("packed", xp, yp, lens, None, slice(None)), ("padded", xf, yf, [S] * B, lens, valid))
    first = {}
    for rep in range(4):
        for name, x, y, seq_lens, valid_lens, rows in cases:
            for call in range(6):
                y.fill_(float("nan"))
                with torch.cuda.stream(stream):
                    model.run_batch(y, x, seq_lens, valid_lens=valid_lens, stream=stream)
                torch.cuda.synchronize()
                model.check()
                if name not in first:
                    first[name] = y[rows].clone()
                    assert torch.isfinite(first[name]).all()
                assert torch.equal(y[rows], first[name]), f"{name} rep {rep} call {call}"


def test_model_argument_checks(et, orc):
    d, H, dff = 128, 2, 256
    lin, ln = make_layer(orc, d, dff, 0.5, seed=40)
    enc = build_encoder(et, et.KIND_TILE, lin, ln, d, 64, H, 64)
    lin2, ln2 = make_layer(orc, 256, 512, 0.5, seed=41)
    other = build_encoder(et, et.KIND_TILE, lin2, ln2, 256, 64, 4, 64)
    with pytest.raises(et.EtError):
        et.Model([enc, other])          # d_model differs
    with pytest.raises(et.EtError):
        et.Model([enc, enc])            # the same layer twice
    model = et.Model([enc])
    with pytest.raises(et.EtError):
        et.Model([enc])                 # already consumed
    x = torch.zeros((64, d), dtype=torch.float16, device="cuda")
    with pytest.raises(et.EtError):
        model.run_batch(x, x, [-1])
    model.run_batch(x, x, [])           # empty batch is a no-op


def test_ingested_tiles_give_the_masked_dense_product(et, orc):
    rng = np.random.default_rng(11)
    K, N, T = 256, 384, 200
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.1).astype(np.float16)
    rp, ro, data = et.prune_dense_to_tiles(W, 0.6)
    w = et.TileWeight(K, N, T, data, rp, ro, bias)
    X = util.activations(12, (T, K))
    y = torch.zeros((T, N), dtype=torch.float16, device="cuda")
    w.run(y, dev(X))
    torch.cuda.synchronize()
    masked = np.zeros((N, K), np.float32)
    for r in range(N // 16):
        for t in range(rp[r], rp[r + 1]):
            masked[r * 16:(r + 1) * 16, ro[t]:ro[t] + 16] = W[r * 16:(r + 1) * 16, ro[t]:ro[t] + 16]
    want = X.astype(np.float32) @ masked.T + bias.astype(np.float32)
    util.assert_close(host(y), want, what="ingested tile weight")
    # dropped tiles are the smallest ones
    kept = int((N // 16) * (K // 16) * 0.4)
    assert len(ro) == kept


def test_ingested_rows_through_row_linear(et, orc):
    rng = np.random.default_rng(13)
    K, N, H, T = 128, 256, 4, 96
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.1).astype(np.float16)
    ids = et.select_rows_magnitude([W], H, 0.5)
    wc, bc = et.compact_rows(W, bias, ids)
    rw = et.RowWeight(K, N, T, wc, ids, bc, H)
    X = util.activations(14, (T, K))
    y = torch.zeros((T, rw.nrow), dtype=torch.float16, device="cuda")
    rw.run(y, dev(X))
    torch.cuda.synchronize()
    want = X.astype(np.float32) @ W[ids].astype(np.float32).T + bias[ids].astype(np.float32)
    util.assert_close(host(y)[:, :len(ids)], want, what="ingested row weight")
    assert rw.head_ptr.tolist() == et.build_head_ptr(ids, H, N).tolist()
