#!/usr/bin/env python
"""Generates tests/golden/reference_kernels.npz: outputs of the reference project's own CUDA kernels (compiled
unchanged from the reference checkout into oracle/_ref/libet_ref.so) on small seeded inputs.

The reference ships no golden vectors and has no CPU path, so these are made by running its kernels on a B200:

    python tests/golden/make_golden.py            # on a machine with a GPU and oracle/_ref/libet_ref.so

The inputs are not stored: tests/test_golden_cpu.py regenerates them from the seeds recorded here (tests/util.py
generators) and checks the CPU oracle against the stored outputs, so the oracle is pinned against the reference
on every run of the CPU suite."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import oracle_lib, util  # noqa: E402

CASES = {
    "ln_v1": dict(num=48, size=768, seed=101),        # the reference's first LayerNorm kernel (size <= 768 path)
    "ln_v2": dict(num=32, size=1024, seed=102),       # its second kernel
    "tile": dict(T=256, K=256, N=256, sparsity=0.5, seed=103),   # M = K, the only shape its tile kernel indexes correctly
    "otf": dict(L=64, d=128, H=2, seed=104, std=0.5),
    "sharedqk": dict(L=64, d=128, H=2, seed=105, std=0.5),
}
LOG2E = 1.4426950408889634


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def p(t):
    return ctypes.c_void_p(t.data_ptr())


def ln_inputs(c):
    x, s = util.activations(c["seed"], (c["num"], c["size"])), util.activations(c["seed"] + 1, (c["num"], c["size"]))
    g = (1.0 + util.weights(c["seed"] + 2, (c["size"],), 0.2).astype(np.float32)).astype(np.float16)
    b = util.weights(c["seed"] + 3, (c["size"],), 0.2)
    return x, s, g, b


def tile_inputs(orc, c):
    rp, ro, data, bias = util.make_tile_linear(orc, c["K"], c["N"], c["sparsity"], seed=c["seed"], bias_std=0.05)
    return rp, ro, data, bias, util.activations(c["seed"] + 1, (c["T"], c["K"]))


def qkv_inputs(c):
    return tuple((util.activations(c["seed"] + i, (c["L"], c["d"])).astype(np.float32) * c["std"]).astype(np.float16)
                 for i in range(3))


def main():
    import torch
    ref = oracle_lib.load_ref()
    if ref is None or not torch.cuda.is_available():
        raise SystemExit("needs a GPU and oracle/_ref/libet_ref.so (make -C oracle with the reference checkout present)")
    orc = oracle_lib.load()
    out = {}
    for name in ("ln_v1", "ln_v2"):
        c = CASES[name]
        x, s, g, b = ln_inputs(c)
        xd, sd, gd, bd = dev(x), dev(s), dev(g), dev(b)
        assert ref.ref_skip_layernorm(p(xd), p(sd), p(gd), p(bd), c["num"], c["size"], None) == 0
        torch.cuda.synchronize()
        out[name] = xd.cpu().numpy()
    c = CASES["tile"]
    rp, ro, data, bias, X = tile_inputs(orc, c)
    for gelu in (0, 1):
        Y = torch.zeros((c["T"], c["N"]), dtype=torch.float16, device="cuda")
        t = [dev(a) for a in (X, rp, ro, data, bias)]
        assert ref.ref_tile_spmm(p(Y), p(t[0]), p(t[1]), p(t[2]), p(t[3]), c["T"], c["N"], c["K"], p(t[4]), gelu, None) == 0
        torch.cuda.synchronize()
        out["tile_gelu" if gelu else "tile"] = Y.cpu().numpy()
    c = CASES["otf"]
    Q, K, V = qkv_inputs(c)
    Qd, Kd, Vd = dev(Q), dev(K), dev(V)
    Md = torch.zeros((c["L"], c["L"]), dtype=torch.float16, device="cuda")
    for key, scale in (("otf_true_softmax", LOG2E / np.sqrt(c["d"] // c["H"])), ("otf_as_shipped", -1.0)):
        Z = torch.zeros((c["L"], c["d"]), dtype=torch.float16, device="cuda")
        assert ref.ref_otf_attention(p(Z), p(Qd), p(Kd), p(Vd), p(Md), c["L"], c["d"], c["H"], ctypes.c_float(scale), None) == 0
        torch.cuda.synchronize()
        out[key] = Z.cpu().numpy()
    c = CASES["sharedqk"]
    Q, K, V = qkv_inputs(c)
    S = (orc.scores(Q, K, c["d"], c["H"]) * LOG2E).astype(np.float16)   # base-2 kernel: scores pre-scaled by log2 e
    Sd, Vd = dev(S), dev(V)
    Md = torch.zeros((c["L"], c["L"]), dtype=torch.float16, device="cuda")
    Z = torch.zeros((c["L"], c["d"]), dtype=torch.float16, device="cuda")
    assert ref.ref_sharedqk_attention(p(Z), p(Sd), p(Vd), p(Md), c["L"], c["d"], c["H"]) == 0
    torch.cuda.synchronize()
    out["sharedqk"] = Z.cpu().numpy()
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz")
    np.savez_compressed(dst, **out)
    extra = os.environ.get("ET_GOLDEN_COPY_DIR")   # optional second copy (e.g. a folder that is carried back from a remote run)
    if extra and os.path.isdir(extra):
        np.savez_compressed(os.path.join(extra, "reference_kernels.npz"), **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
