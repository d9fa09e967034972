#!/usr/bin/env python
"""One kernel at a time on inputs larger than L2: prints the achieved rate from CUDA events.

    python et_b200/examples/kernel_cases.py {gemm|gemm_large|attention|attention512|attention_mma|layernorm|softmax} [launches]

`attention_mma` is `attention` with the lengths given only on the device, which the tcgen05 kernel declines
(it needs the longest length on the host), so the mma.sync kernel runs.

Sized for profiling too (a few hundred MB on the device, a handful of launches):
    ncu --set full --clock-control none -k regex:<kernel> -s 3 -c 2 -o out python et_b200/examples/kernel_cases.py gemm
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import et_b200 as et  # noqa: E402


def timed(fn, n):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e-3


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 5
    if case in ("gemm", "gemm_large"):
        # gemm: the base model's FFN1 shape; gemm_large: BERT-large's (in 1024, out 4096, 80 % of the tiles pruned)
        T, K, N, sparsity = (16384, 768, 3072, 0.75) if case == "gemm" else (16384, 1024, 4096, 0.8)
        rp, ro = et.gen_sparse_tile_mat(N, K, sparsity, 7, bernoulli=True)
        rng = np.random.default_rng(0)
        data = (rng.standard_normal((len(ro), 256), dtype=np.float32) * 0.02).astype(np.float16)
        w = et.TileWeight(K, N, T, data, rp, ro, np.zeros(N, np.float16))
        x = torch.randn((T, K), device="cuda").half()
        y = torch.zeros((T, N), dtype=torch.float16, device="cuda")
        s = timed(lambda: w.run(y, x), n)
        flops = 2.0 * T * 256 * len(ro)
        print(f"tile GEMM T={T} K={K} N={N} kept tiles {len(ro)} ({len(ro) / (N // 16 * K // 16):.3f}): {s * 1e6:.1f} us, "
              f"{flops / s / 1e12:.1f} TFLOP/s on kept tiles, {flops / s / 1e12 / (len(ro) / (N // 16 * K // 16)):.0f} dense-equivalent; {w.info()}")
    elif case in ("attention", "attention512", "attention_mma"):
        S = 512 if case == "attention512" else 128
        B, d, H = (64, 768, 12) if S == 512 else (256, 768, 12)
        q, k, v = (torch.randn((B * S, d), device="cuda").half() for _ in range(3))
        o = torch.zeros_like(q)
        if case == "attention_mma":
            cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
            s = timed(lambda: et.attention_batch(o, q, k, v, d, H, cu_seqlens=cu, batch=B), n)
        else:
            s = timed(lambda: et.attention_batch(o, q, k, v, d, H, batch=B, uniform_len=S), n)
        flops = 4.0 * S * S * d * B
        print(f"attention B={B} S={S} d={d} H={H}: {s * 1e6:.1f} us, {flops / s / 1e12:.1f} TFLOP/s")
    elif case == "layernorm":
        rows, dm = 131072, 1024
        a, b = torch.randn((rows, dm), device="cuda").half(), torch.randn((rows, dm), device="cuda").half()
        g, be = torch.ones(dm, dtype=torch.float16, device="cuda"), torch.zeros(dm, dtype=torch.float16, device="cuda")
        s = timed(lambda: et.skip_layernorm(a, b, g, be), n)
        print(f"skip-LayerNorm {rows}x{dm}: {s * 1e6:.1f} us, {6.0 * rows * dm / s / 1e9:.0f} GB/s (6 bytes per element)")
    elif case == "softmax":
        nmat, L = 1024, 512
        sc = torch.randn((nmat, L, L), device="cuda").half()
        m = torch.zeros((L, L), dtype=torch.float16, device="cuda")
        s = timed(lambda: et.softmax_mask(sc, m), n)
        print(f"mask+softmax {nmat}x{L}x{L}: {s * 1e6:.1f} us, {4.0 * nmat * L * L / s / 1e9:.0f} GB/s (4 bytes per score)")
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main()
