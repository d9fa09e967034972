"""Pins the CPU oracle against outputs of the reference project's own CUDA kernels, stored in
tests/golden/reference_kernels.npz (made on a B200 by tests/golden/make_golden.py). Inputs are regenerated from
the seeds in that script. The reference accumulates in fp16, so the bounds are looser than the gate for the new
kernels (which is checked against the oracle in the GPU suite)."""
import os

import numpy as np
import pytest

from tests import util
from tests.golden import make_golden as mg
from tests.oracle_lib import REF_COMPAT

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz")


@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLDEN):
        pytest.fail("tests/golden/reference_kernels.npz is missing: run tests/golden/make_golden.py on a GPU box")
    return np.load(GOLDEN)


@pytest.mark.parametrize("name", ["ln_v1", "ln_v2"])
def test_oracle_layernorm_matches_reference_kernel_output(orc, gold, name):
    x, s, g, b = mg.ln_inputs(mg.CASES[name])
    util.assert_close(gold[name].astype(np.float32), orc.skip_layernorm(x, s, g, b), max_abs=6e-2, mean_abs=6e-3,
                      what=f"reference {name} vs oracle")


@pytest.mark.parametrize("gelu", [False, True])
def test_oracle_tile_linear_matches_reference_kernel_output(orc, gold, gelu):
    c = mg.CASES["tile"]
    rp, ro, data, bias, X = mg.tile_inputs(orc, c)
    want = orc.tile_linear(X, rp, ro, data, bias, c["N"], gelu=gelu)
    util.assert_close(gold["tile_gelu" if gelu else "tile"].astype(np.float32), want, max_abs=4e-2, mean_abs=4e-3,
                      what="reference tile GEMM vs oracle")


def test_oracle_attention_matches_reference_kernel_output(orc, gold):
    c = mg.CASES["otf"]
    Q, K, V = mg.qkv_inputs(c)
    # with log2(e) folded into its scale the reference's base-2 kernel computes a true softmax
    util.assert_close(gold["otf_true_softmax"].astype(np.float32), orc.attention(Q, K, V, [c["L"]], c["d"], c["H"]),
                      max_abs=6e-2, mean_abs=6e-3, what="reference OTF vs oracle")
    # as shipped (base 2, row maximum floored at 0): the oracle's compatibility mode restates it
    util.assert_close(gold["otf_as_shipped"].astype(np.float32),
                      orc.attention(Q, K, V, [c["L"]], c["d"], c["H"], flags=REF_COMPAT),
                      max_abs=6e-2, mean_abs=6e-3, what="reference OTF as shipped vs compat oracle")


def test_oracle_sharedqk_matches_reference_kernel_output(orc, gold):
    c = mg.CASES["sharedqk"]
    Q, K, V = mg.qkv_inputs(c)
    util.assert_close(gold["sharedqk"].astype(np.float32), orc.attention(Q, K, V, [c["L"]], c["d"], c["H"]),
                      max_abs=6e-2, mean_abs=6e-3, what="reference sharedQK vs oracle")
