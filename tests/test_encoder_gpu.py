"""GPU parity tests of the encoder layer objects (C ABI) against the CPU oracle at the workload configs
(reduced where the oracle would take too long), plus size-independent properties at full size."""
import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.float().cpu().numpy()


@pytest.fixture(scope="module")
def et():
    import et_b200
    et_b200.lib()
    return et_b200


def make_layer(orc, d, dff, sparsity, seed, bernoulli=True, bias_std=0.02, unit_scale=False):
    """unit_scale: weight std 1/sqrt(kept inputs) instead of 0.02, so that every sub-layer's output is as large as
    the residual it is added to (with std 0.02 the attention and FFN branches are a few per cent of the residual
    and an error in them hides below the tolerance)."""
    shapes = {"q": (d, d), "k": (d, d), "v": (d, d), "o": (d, d), "ffn1": (d, dff), "ffn2": (dff, d)}
    lin = {}
    for i, (name, (K, N)) in enumerate(shapes.items()):
        std = 1.0 / np.sqrt(K * max(1.0 - sparsity, 1e-3)) if unit_scale else 0.02
        rp, ro, data, bias = util.make_tile_linear(orc, K, N, sparsity, seed + 10 * i, bernoulli, bias_std, std=std)
        lin[name] = (rp, ro, data, bias, N, K)
    g = [(1.0 + util.weights(seed + 100 + j, (d,), 0.1).astype(np.float32)).astype(np.float16) for j in range(2)]
    b = [util.weights(seed + 110 + j, (d,), 0.1) for j in range(2)]
    return lin, ((g[0], b[0]), (g[1], b[1]))


def tile_weights(et, lin, size):
    out = {}
    for name, (rp, ro, data, bias, N, K) in lin.items():
        out[name] = et.TileWeight(K, N, size, data, rp, ro, bias, is_gelu=(name == "ffn1"))
    return out


def build_encoder(et, kind, lin, ln, d, S, H, size, buffer=None, mask=None):
    w = tile_weights(et, lin, size)
    return et.Encoder(kind, d, S, H, buffer, w["q"], w["k"], w["v"], w["o"], w["ffn1"], w["ffn2"],
                      (ln[0][0], ln[0][1], ln[1][0], ln[1][1]), mask)


def orc_lin(lin):
    return {k: v[:5] for k, v in lin.items()}


@pytest.mark.parametrize("S,sparsity", [(128, 0.0), (128, 0.5), (64, 0.9)])
def test_encoder_tile_single_sequence_run(et, orc, S, sparsity):
    """Config 1 (dense base layer, B=1, S=128) and pruned variants through Encoder_tile::run; out aliases in."""
    d, H, dff = 768, 12, 3072
    lin, ln = make_layer(orc, d, dff, sparsity, seed=1, bernoulli=False)
    mask = np.zeros((S, S), dtype=np.float16)
    buf = torch.zeros(et.encoder_buffer_size(et.KIND_TILE, d, S, H) // 2, dtype=torch.float16, device="cuda")
    enc = build_encoder(et, et.KIND_TILE, lin, ln, d, S, H, S, buffer=buf, mask=mask)
    X = util.activations(7, (S, d))
    want = orc.encoder_layer(X, orc_lin(lin), ln, [S], d, H, mask=mask.astype(np.float32))
    x = dev(X)
    enc.run(x, x)
    torch.cuda.synchronize()
    util.assert_close(host(x), want, what=f"Encoder_tile S={S} sparsity={sparsity}")


@pytest.mark.parametrize("sparsity", [0.5, 0.75, 0.9])
def test_encoder_tile_batch_config2(et, orc, sparsity):
    """Config 2: B=16, S=128, tile-pruned base layer, Bernoulli tile mask."""
    d, H, dff, B, S = 768, 12, 3072, 16, 128
    lin, ln = make_layer(orc, d, dff, sparsity, seed=2)
    enc = build_encoder(et, et.KIND_TILE, lin, ln, d, S, H, B * S)
    X = util.activations(8, (B * S, d))
    want = orc.encoder_layer(X, orc_lin(lin), ln, [S] * B, d, H)
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, d, B * S, B, S, H) // 2,
                          dtype=torch.float16, device="cuda")
    out = torch.zeros((B * S, d), dtype=torch.float16, device="cuda")
    enc.run_batch(out, dev(X), [S] * B, scratch)
    torch.cuda.synchronize()
    util.assert_close(host(out), want, what=f"config 2 sparsity={sparsity}")


def test_encoder_tile_batch_config2_packed_for_throughput(et, orc):
    """Config 2 with the weights packed under the throughput goal, several calls in a row so that the direct run,
    the graph capture and the replays are all compared with the oracle."""
    d, H, dff, B, S = 768, 12, 3072, 16, 128
    lin, ln = make_layer(orc, d, dff, 0.75, seed=12)
    et.set_tuning_goal("throughput")
    try:
        enc = build_encoder(et, et.KIND_TILE, lin, ln, d, S, H, B * S)
    finally:
        et.set_tuning_goal("latency")
    X = util.activations(18, (B * S, d))
    want = orc.encoder_layer(X, orc_lin(lin), ln, [S] * B, d, H)
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, d, B * S, B, S, H) // 2,
                          dtype=torch.float16, device="cuda")
    x = dev(X)
    side = torch.cuda.Stream()
    for call in range(4):
        out = torch.full((B * S, d), float("nan"), dtype=torch.float16, device="cuda")
        with torch.cuda.stream(side):
            enc.run_batch(out, x, [S] * B, scratch)
        torch.cuda.synchronize()
        util.assert_close(host(out), want, what=f"config 2, throughput packing, call {call}")
    enc.check()


def test_run_batch_alternating_batch_sizes_keeps_replayed_graphs_valid(et, orc):
    """Variable-length batches of 4, then 8, then the first 4 again, three or more calls each: the device array of
    lengths grows in between, and the graphs recorded before that must not be replayed against the old array."""
    d, H, dff = 768, 12, 3072
    lin, ln = make_layer(orc, d, dff, 0.75, seed=13)
    lens_a = [40, 128, 17, 96]
    lens_b = [64, 33, 128, 90, 5, 77, 128, 100]
    # a third shape that needs more than the first allocation's 64 entries
    lens_c = [16 + (7 * i) % 48 for i in range(40)]
    enc = build_encoder(et, et.KIND_LENGTH, lin, ln, d, 128, H, sum(lens_b))
    stream = torch.cuda.Stream()
    cases = {}
    for name, lens in (("a", lens_a), ("b", lens_b), ("c", lens_c)):
        T = sum(lens)
        X = util.activations(30 + len(lens), (T, d))
        cases[name] = (lens, dev(X), torch.zeros((T, d), dtype=torch.float16, device="cuda"),
                       orc.encoder_layer(X, orc_lin(lin), ln, lens, d, H))
    Tmax = max(sum(c[0]) for c in cases.values())
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_LENGTH, d, Tmax, 40, 128, H) // 2,
                          dtype=torch.float16, device="cuda")
    for name in ("a", "a", "a", "b", "b", "b", "a", "a", "c", "c", "c", "a", "b", "a"):
        lens, x, out, want = cases[name]
        out.fill_(float("nan"))
        with torch.cuda.stream(stream):
            enc.run_batch(out, x, lens, scratch)
        torch.cuda.synchronize()
        util.assert_close(host(out), want, what=f"alternating varlen batches, case {name}")
    enc.check()


def test_encoder_length_varlen_equals_padded_and_oracle(et, orc):
    """Config 4 mechanics at reduced size: variable lengths (not multiples of 16) vs the same batch padded to
    max length with key padding; both match the oracle on the valid tokens; materialised-score path too."""
    d, H, dff = 768, 12, 3072
    lens = [33, 128, 77, 256, 32, 190]
    B, S = len(lens), 256
    lin, ln = make_layer(orc, d, dff, 0.75, seed=3)
    T = sum(lens)
    X = util.activations(9, (T, d))
    want = orc.encoder_layer(X, orc_lin(lin), ln, lens, d, H)
    enc = build_encoder(et, et.KIND_LENGTH, lin, ln, d, S, H, T)
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_LENGTH, d, B * S, B, S, H) // 2,
                          dtype=torch.float16, device="cuda")
    out = torch.zeros((T, d), dtype=torch.float16, device="cuda")
    enc.run_batch(out, dev(X), lens, scratch)
    torch.cuda.synchronize()
    util.assert_close(host(out), want, what="varlen encoder")
    # padded: every sequence occupies S rows, padding rows hold zeros, keys beyond the length are masked
    Xp = np.zeros((B * S, d), dtype=np.float16)
    rows = np.concatenate([np.arange(b * S, b * S + lens[b]) for b in range(B)])
    Xp[rows] = X
    outp = torch.zeros((B * S, d), dtype=torch.float16, device="cuda")
    enc.run_batch(outp, dev(Xp), [S] * B, scratch, valid_lens=lens)
    torch.cuda.synchronize()
    got_valid = host(outp)[rows]
    util.assert_close(got_valid, want, what="padded encoder, valid rows")
    assert np.abs(got_valid - host(out)).max() <= 2e-3   # same kernels, same arithmetic per token
    # the reference's structure: scores materialised in HBM, equal lengths
    enc.set_materialize_scores(True)
    outm = torch.zeros((B * S, d), dtype=torch.float16, device="cuda")
    enc.run_batch(outm, dev(Xp), [S] * B, scratch, valid_lens=lens)
    torch.cuda.synchronize()
    util.assert_close(host(outm)[rows], want, what="materialised-score encoder, valid rows")


def test_encoder_prune_v_and_qkv(et, orc):
    """Config 3 mechanics at reduced batch: row-pruned V (reference ctor) and row-pruned Q/K/V (extension),
    FFN 75 % tile-pruned."""
    d, H, dff, B, S = 768, 12, 3072, 4, 256
    lin, ln = make_layer(orc, d, dff, 0.75, seed=4)
    X = util.activations(10, (B * S, d))
    row_id = orc.gen_sparse_row_mat(d, 0.5, seed=12, nhead=H)
    hp = orc.head_ptr(row_id, H, d)
    Wr = {n: util.weights(200 + i, (len(row_id), d)) for i, n in enumerate("qkv")}
    br = {n: util.weights(210 + i, (len(row_id),), 0.02) for i, n in enumerate("qkv")}
    ol = orc_lin(lin)

    def oracle(prune_qk):
        Xf = X.astype(np.float32)
        if prune_qk:
            q = orc.row_linear(Xf, Wr["q"], br["q"])
            k = orc.row_linear(Xf, Wr["k"], br["k"])
        else:
            q = orc.tile_linear(Xf, *ol["q"][:4], ol["q"][4])
            k = orc.tile_linear(Xf, *ol["k"][:4], ol["k"][4])
        v = orc.row_linear(Xf, Wr["v"], br["v"])
        z = orc.attention(q, k, v, [S] * B, d, H, qk_head_ptr=hp if prune_qk else None, v_col_id=row_id,
                          v_head_ptr=hp)
        a = orc.tile_linear(z, *ol["o"][:4], ol["o"][4])
        h1 = orc.skip_layernorm(a, Xf, *ln[0])
        f = orc.tile_linear(h1, *ol["ffn1"][:4], ol["ffn1"][4], gelu=True)
        y = orc.tile_linear(f, *ol["ffn2"][:4], ol["ffn2"][4])
        return orc.skip_layernorm(y, h1, *ln[1])

    lnp = (ln[0][0], ln[0][1], ln[1][0], ln[1][1])
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_PRUNE, d, B * S, B, S, H) // 2,
                          dtype=torch.float16, device="cuda")
    for prune_qk in (False, True):
        w = tile_weights(et, lin, B * S)
        rv = et.RowWeight(d, d, B * S, Wr["v"], row_id, br["v"], H)
        if prune_qk:
            rq = et.RowWeight(d, d, B * S, Wr["q"], row_id, br["q"], H)
            rk = et.RowWeight(d, d, B * S, Wr["k"], row_id, br["k"], H)
            enc = et.Encoder(et.KIND_PRUNE_QKV, d, S, H, None, rq, rk, rv, w["o"], w["ffn1"], w["ffn2"], lnp)
        else:
            enc = et.Encoder(et.KIND_PRUNE, d, S, H, None, w["q"], w["k"], rv, w["o"], w["ffn1"], w["ffn2"], lnp)
        out = torch.zeros((B * S, d), dtype=torch.float16, device="cuda")
        enc.run_batch(out, dev(X), [S] * B, scratch)
        torch.cuda.synchronize()
        util.assert_close(host(out), oracle(prune_qk), what=f"Encoder_prune prune_qk={prune_qk}")


def test_encoder_kinds_with_unit_scale_weights(et, orc):
    """Every encoder kind with weights scaled so that the attention and FFN branches are as large as the residual:
    the operand pitches and head windows that the layer hands to the attention kernels (fused Q|K|V buffers,
    compact row-pruned operands, materialised scores) all have to be right for this to pass."""
    d, H, dff, S = 256, 4, 1024, 128
    lin, ln = make_layer(orc, d, dff, 0.5, seed=70, unit_scale=True)
    ol = orc_lin(lin)
    lnp = (ln[0][0], ln[0][1], ln[1][0], ln[1][1])
    lens = [128, 37, 90]
    T = sum(lens)
    X = util.activations(71, (T, d))
    want = orc.encoder_layer(X, ol, ln, lens, d, H)
    tol = dict(max_abs=4e-2, mean_abs=4e-3)   # fp16 storage of O(1) intermediates through five fused stages
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_LENGTH, d, 3 * S, 3, S, H) // 2, dtype=torch.float16, device="cuda")
    # tile layer, variable lengths (tensor-core attention, fused Q|K|V)
    enc = build_encoder(et, et.KIND_LENGTH, lin, ln, d, S, H, T)
    out = torch.zeros((T, d), dtype=torch.float16, device="cuda")
    enc.run_batch(out, dev(X), lens, scratch)
    torch.cuda.synchronize()
    util.assert_close(host(out), want, what="unit-scale weights, varlen", **tol)
    # padded with key padding, on the fly and through materialised scores
    Xp = np.zeros((3 * S, d), dtype=np.float16)
    rows = np.concatenate([np.arange(b * S, b * S + lens[b]) for b in range(3)])
    Xp[rows] = X
    for mat in (False, True):
        enc.set_materialize_scores(mat)
        outp = torch.zeros((3 * S, d), dtype=torch.float16, device="cuda")
        enc.run_batch(outp, dev(Xp), [S] * 3, scratch, valid_lens=lens)
        torch.cuda.synchronize()
        util.assert_close(host(outp)[rows], want, what=f"unit-scale weights, padded, materialised scores {mat}", **tol)
    # row-pruned V, and row-pruned Q, K and V
    row_id = orc.gen_sparse_row_mat(d, 0.5, seed=72, nhead=H)
    hp = orc.head_ptr(row_id, H, d)
    std = 1.0 / np.sqrt(d)
    Wr = {n: util.weights(300 + i, (len(row_id), d), std) for i, n in enumerate("qkv")}
    br = {n: util.weights(310 + i, (len(row_id),), 0.02) for i, n in enumerate("qkv")}
    Xf = X.astype(np.float32)
    for prune_qk in (False, True):
        if prune_qk:
            q, k = orc.row_linear(Xf, Wr["q"], br["q"]), orc.row_linear(Xf, Wr["k"], br["k"])
        else:
            q, k = orc.tile_linear(Xf, *ol["q"][:4], ol["q"][4]), orc.tile_linear(Xf, *ol["k"][:4], ol["k"][4])
        v = orc.row_linear(Xf, Wr["v"], br["v"])
        z = orc.attention(q, k, v, lens, d, H, qk_head_ptr=hp if prune_qk else None, v_col_id=row_id, v_head_ptr=hp)
        a = orc.tile_linear(z, *ol["o"][:4], ol["o"][4])
        h1 = orc.skip_layernorm(a, Xf, *ln[0])
        f = orc.tile_linear(h1, *ol["ffn1"][:4], ol["ffn1"][4], gelu=True)
        wantp = orc.skip_layernorm(orc.tile_linear(f, *ol["ffn2"][:4], ol["ffn2"][4]), h1, *ln[1])
        w = tile_weights(et, lin, T)
        rv = et.RowWeight(d, d, T, Wr["v"], row_id, br["v"], H)
        if prune_qk:
            encp = et.Encoder(et.KIND_PRUNE_QKV, d, S, H, None, et.RowWeight(d, d, T, Wr["q"], row_id, br["q"], H),
                              et.RowWeight(d, d, T, Wr["k"], row_id, br["k"], H), rv, w["o"], w["ffn1"], w["ffn2"], lnp)
        else:
            encp = et.Encoder(et.KIND_PRUNE, d, S, H, None, w["q"], w["k"], rv, w["o"], w["ffn1"], w["ffn2"], lnp)
        outq = torch.zeros((T, d), dtype=torch.float16, device="cuda")
        encp.run_batch(outq, dev(X), lens, scratch)
        torch.cuda.synchronize()
        util.assert_close(host(outq), wantp, what=f"unit-scale weights, row-pruned, prune_qk={prune_qk}", **tol)
        encp.check()


def test_bert_large_layer_properties_at_full_slab(et, orc):
    """Config 5 shapes (d=1024, H=16, ff=4096, S=512, 80 % pruned): oracle parity on 2 sequences, and at a
    larger batch the size-independent property that every sequence is processed independently of its
    neighbours (batch of B equals B batches of 1, bit for bit)."""
    d, H, dff, S = 1024, 16, 4096, 512
    lin, ln = make_layer(orc, d, dff, 0.8, seed=5)
    B = 8
    X = util.activations(11, (B * S, d))
    enc = build_encoder(et, et.KIND_TILE, lin, ln, d, S, H, B * S)
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, d, B * S, B, S, H) // 2,
                          dtype=torch.float16, device="cuda")
    out = torch.zeros((B * S, d), dtype=torch.float16, device="cuda")
    xd = dev(X)
    enc.run_batch(out, xd, [S] * B, scratch)
    torch.cuda.synchronize()
    want = orc.encoder_layer(X[:2 * S], orc_lin(lin), ln, [S, S], d, H)
    util.assert_close(host(out)[:2 * S], want, what="BERT-large layer, 2 sequences")
    one = torch.zeros((S, d), dtype=torch.float16, device="cuda")
    for b in (0, 3, 7):
        enc.run_batch(one, xd[b * S:(b + 1) * S], [S], scratch)
        torch.cuda.synchronize()
        assert torch.equal(one, out[b * S:(b + 1) * S])


def test_encoder_rejects_bad_arguments(et, orc):
    d, H, dff, S = 128, 2, 512, 32
    lin, ln = make_layer(orc, d, dff, 0.5, seed=6)
    enc = build_encoder(et, et.KIND_TILE, lin, ln, d, S, H, S)
    x = torch.zeros((S, d), dtype=torch.float16, device="cuda")
    with pytest.raises(et.EtError):      # created without a scratch buffer: run() refuses
        enc.run(x, x)
    small = torch.zeros(16, dtype=torch.float16, device="cuda")
    with pytest.raises(et.EtError):      # scratch too small
        enc.run_batch(x, x, [S], small)
    with pytest.raises(et.EtError):      # negative length
        enc.run_batch(x, x, [-1], small)
    with pytest.raises(et.EtError):
        enc.set_materialize_scores(True)  # only the length encoder has that path


def test_run_batch_on_the_legacy_stream_and_on_a_side_stream_agree(et, orc):
    """On the legacy default stream the layer runs on a stream of the encoder (ordered by events) so that the graph
    replay still engages; results are bit-identical to a caller-provided stream, and ordered with the caller's
    other work on the legacy stream."""
    d, H, dff, B, S = 256, 4, 512, 3, 64
    lin, ln = make_layer(orc, d, dff, 0.5, seed=61)
    enc = build_encoder(et, et.KIND_TILE, lin, ln, d, S, H, B * S)
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, d, B * S, B, S, H) // 2, dtype=torch.float16, device="cuda")
    x = dev(util.activations(62, (B * S, d)))
    side = torch.cuda.Stream()
    ref_out = torch.zeros_like(x)
    with torch.cuda.stream(side):
        enc.run_batch(ref_out, x, [S] * B, scratch)
    side.synchronize()
    for call in range(4):            # direct, captured, replayed, replayed
        xin = x.clone()              # produced on the legacy stream right before the call
        out = torch.zeros_like(x)
        enc.run_batch(out, xin, [S] * B, scratch)
        doubled = out * 2            # consumed on the legacy stream right after the call
        torch.cuda.synchronize()
        assert torch.equal(out, ref_out), f"call {call}"
        assert torch.equal(doubled, ref_out * 2)
