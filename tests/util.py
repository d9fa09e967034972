"""Seeded synthetic inputs and the tolerance check shared by the tests."""
import numpy as np

MAX_ABS_TOL = 2e-2   # fp16 result against the fp32 oracle
MEAN_ABS_TOL = 2e-3


def rng(seed):
    return np.random.default_rng(seed)


def activations(seed, shape):
    """~N(0,1), rounded to fp16."""
    return rng(seed).standard_normal(shape, dtype=np.float32).astype(np.float16)


def weights(seed, shape, std=0.02):
    return (rng(seed).standard_normal(shape, dtype=np.float32) * std).astype(np.float16)


def make_tile_linear(orc, in_feat, out_feat, sparsity, seed, bernoulli=True, bias_std=0.0,
                     std=0.02):
    """(row_ptr, row_offset, data[ntile,256] fp16, bias[out_feat] fp16) in the reference's tile format."""
    row_ptr, row_offset = orc.gen_sparse_tile_mat(out_feat, in_feat, sparsity, seed, bernoulli)
    data = weights(seed + 1, (len(row_offset), 256), std)
    if bias_std > 0:
        bias = weights(seed + 2, (out_feat,), bias_std)
    else:
        bias = np.zeros(out_feat, dtype=np.float16)
    return row_ptr, row_offset, data, bias


def assert_close(got, want, max_abs=MAX_ABS_TOL, mean_abs=MEAN_ABS_TOL, what=""):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    d = np.abs(got - want)
    mx, mn = float(d.max()) if d.size else 0.0, float(d.mean()) if d.size else 0.0
    assert mx <= max_abs and mn <= mean_abs, f"{what}: max-abs {mx:.4g} (tol {max_abs}), mean-abs {mn:.4g} (tol {mean_abs})"
    return mx, mn
