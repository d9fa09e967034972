"""Magnitude-based ingestion of dense weights into the two pruned formats, and the length-bucketing scheduler:
host logic, checked against numpy restatements (no GPU)."""
import numpy as np
import pytest

import et_b200 as et
from et_b200 import scheduler


def tile_scores(w):
    o, i = w.shape
    t = w.astype(np.float64).reshape(o // 16, 16, i // 16, 16)
    return (t * t).sum(axis=(1, 3))


@pytest.mark.parametrize("shape,sparsity", [((64, 96), 0.5), ((128, 64), 0.75), ((32, 32), 0.0), ((48, 80), 1.0)])
def test_prune_dense_to_tiles_matches_numpy(shape, sparsity):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal(shape) * 0.05).astype(np.float16)
    rp, ro, data = et.prune_dense_to_tiles(w, sparsity)
    sc = tile_scores(w)
    total = sc.size
    kept = int(total * (1.0 - sparsity))
    order = np.argsort(-sc.ravel(), kind="stable")[:kept]
    keep = np.zeros(total, bool)
    keep[order] = True
    keep = keep.reshape(sc.shape)
    assert rp[-1] == kept and len(ro) == kept
    want_rp = np.concatenate([[0], np.cumsum(keep.sum(axis=1))]).astype(np.int32)
    assert np.array_equal(rp, want_rp)
    t = 0
    for r in range(sc.shape[0]):
        for c in np.nonzero(keep[r])[0]:
            assert ro[t] == c * 16
            assert np.array_equal(data[t].reshape(16, 16), w[r * 16:(r + 1) * 16, c * 16:(c + 1) * 16])
            t += 1


def test_tile_ties_keep_the_lower_index():
    w = np.ones((32, 32), np.float16)   # four tiles of equal norm
    rp, ro, _ = et.prune_dense_to_tiles(w, 0.5)
    assert list(rp) == [0, 2, 2] and list(ro) == [0, 16]


def test_select_and_compact_rows():
    rng = np.random.default_rng(5)
    nhead, out_feat, in_feat = 4, 64, 48
    wq = (rng.standard_normal((out_feat, in_feat)) * 0.1).astype(np.float16)
    wk = (rng.standard_normal((out_feat, in_feat)) * 0.1).astype(np.float16)
    bias = rng.standard_normal(out_feat).astype(np.float16)
    ids = et.select_rows_magnitude([wq, wk], nhead, 0.5)
    hd = out_feat // nhead
    score = (wq.astype(np.float64) ** 2).sum(1) + (wk.astype(np.float64) ** 2).sum(1)
    want = []
    for h in range(nhead):
        idx = np.arange(h * hd, (h + 1) * hd)
        top = idx[np.argsort(-score[idx], kind="stable")[:hd // 2]]
        want += sorted(top.tolist())
    assert ids.tolist() == want
    hp = et.build_head_ptr(ids, nhead, out_feat)
    assert hp.tolist() == [0, 8, 16, 24, 32]
    wc, bc = et.compact_rows(wq, bias, ids)
    assert wc.shape == (32, in_feat)
    assert np.array_equal(wc, wq[ids]) and np.array_equal(bc, bias[ids])
    # an odd count is padded with zero rows
    wc, bc = et.compact_rows(wq, None, ids[:5])
    assert wc.shape == (16, in_feat) and not wc[5:].any() and not bc.any()
    assert np.array_equal(wc[:5], wq[ids[:5]])


def test_every_head_keeps_a_row_at_full_sparsity():
    w = np.random.default_rng(1).standard_normal((32, 16)).astype(np.float16)
    ids = et.select_rows_magnitude([w], 4, 1.0)
    assert len(ids) == 4 and sorted(set(i // 8 for i in ids)) == [0, 1, 2, 3]


def test_ingestion_argument_checks():
    with pytest.raises(et.EtError):
        et.prune_dense_to_tiles(np.zeros((20, 32), np.float16), 0.5)
    with pytest.raises(et.EtError):
        et.select_rows_magnitude([np.zeros((30, 16), np.float16)], 4, 0.5)
    with pytest.raises(et.EtError):
        et.compact_rows(np.zeros((32, 16), np.float16), None, [3, 2])


def test_bucket_by_length_bounds_and_order():
    rng = np.random.default_rng(9)
    lengths = rng.integers(1, 513, size=200).tolist() + [0, 700]
    batches = scheduler.bucket_by_length(lengths, max_tokens=2048, width=64, max_batch=16)
    seen = sorted(i for b in batches for i in b.indices)
    assert seen == [i for i, l in enumerate(lengths) if l > 0]
    for b in batches:
        assert b.indices == sorted(b.indices) and len(b.indices) <= 16
        assert all(scheduler.bucket_ceiling(l, 64) == b.padded_to for l in b.lengths)
        assert b.tokens <= 2048 or len(b.indices) == 1
    assert [b.padded_to for b in batches] == sorted(b.padded_to for b in batches)
    assert scheduler.padding_waste(batches) < 0.25
    outs = [[("r", i) for i in b.indices] for b in batches]
    back = scheduler.restore_order(batches, outs, len(lengths))
    assert back[200] is None and all(back[i] == ("r", i) for i in seen)


def test_bucket_argument_checks():
    with pytest.raises(ValueError):
        scheduler.bucket_by_length([4], 0)
    with pytest.raises(ValueError):
        scheduler.bucket_by_length([-1], 16)
    with pytest.raises(ValueError):
        scheduler.bucket_ceiling(5, 0)
