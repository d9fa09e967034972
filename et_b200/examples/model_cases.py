#!/usr/bin/env python
"""Whole-model cases on synthetic weights: a stack of tile-pruned encoder layers over a batch of sequences.

    python et_b200/examples/model_cases.py varlen   [layers] [batch]   # lengths uniform on [32, 512] vs padded to 512
    python et_b200/examples/model_cases.py large    [layers] [batch]   # BERT-large shape, 512 tokens, tile sparsity 0.8
    python et_b200/examples/model_cases.py bucketed [layers] [requests] # length-bucketed batches of a request stream
    python et_b200/examples/model_cases.py pruned   [layers] [batch]   # attention-aware pruning: half of the Q/K/V rows
                                                                       # of every head, 256 tokens, FFN tile sparsity 0.75

Prints sequences/s and microseconds per layer from CUDA events (model-owned scratch, all layers replayed as one
CUDA graph)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import et_b200 as et  # noqa: E402
from et_b200 import scheduler  # noqa: E402


def tile_weight(rng, K, N, sparsity, tokens, seed, gelu=False):
    rp, ro = et.gen_sparse_tile_mat(N, K, sparsity, seed, bernoulli=True)
    data = (rng.standard_normal((len(ro), 256), dtype=np.float32) * 0.02).astype(np.float16)
    return et.TileWeight(K, N, tokens, data, rp, ro, np.zeros(N, np.float16), is_gelu=gelu)


def make_model(kind, layers, d, heads, ff, sparsity, tokens, max_len):
    rng = np.random.default_rng(0)
    ones, zeros = np.ones(d, np.float16), np.zeros(d, np.float16)
    encs = []
    for i in range(layers):
        w = [tile_weight(rng, d, d, sparsity, tokens, 100 * i + j) for j in range(4)]
        w.append(tile_weight(rng, d, ff, sparsity, tokens, 100 * i + 4, gelu=True))
        w.append(tile_weight(rng, ff, d, sparsity, tokens, 100 * i + 5))
        encs.append(et.Encoder(kind, d, max_len, heads, None, *w, (ones, zeros, ones, zeros)))
    return et.Model(encs)


def timed(fn, n, warm=3):
    for _ in range(warm):
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
    case = sys.argv[1] if len(sys.argv) > 1 else "varlen"
    layers = int(sys.argv[2]) if len(sys.argv) > 2 else 12
    rng = np.random.default_rng(1)
    if case == "varlen":
        batch = int(sys.argv[3]) if len(sys.argv) > 3 else 64
        d, heads, ff = 768, 12, 3072
        lens = rng.integers(32, 513, size=batch).tolist()
        T, Tp = sum(lens), 512 * batch
        model = make_model(et.KIND_LENGTH, layers, d, heads, ff, 0.75, Tp, 512)
        x = torch.randn((T, d), device="cuda").half()
        out = torch.zeros_like(x)
        s = timed(lambda: model.run_batch(out, x, lens), 10)
        xp = torch.randn((Tp, d), device="cuda").half()
        outp = torch.zeros_like(xp)
        sp = timed(lambda: model.run_batch(outp, xp, [512] * batch, valid_lens=lens), 10)
        print(f"{layers} layers, {batch} sequences, lengths U[32,512] ({T} tokens): packed {s * 1e3:.2f} ms "
              f"({batch / s:.0f} seq/s, {s / layers * 1e6:.0f} us/layer); padded to 512 ({Tp} tokens) {sp * 1e3:.2f} ms "
              f"({batch / sp:.0f} seq/s); packed is {sp / s:.2f} x faster")
    elif case == "large":
        batch = int(sys.argv[3]) if len(sys.argv) > 3 else 32
        d, heads, ff, S = 1024, 16, 4096, 512
        T = batch * S
        model = make_model(et.KIND_TILE, layers, d, heads, ff, 0.8, T, S)
        x = torch.randn((T, d), device="cuda").half()
        out = torch.zeros_like(x)
        s = timed(lambda: model.run_batch(out, x, [S] * batch), 5)
        print(f"{layers} layers large, {batch} x {S} tokens, tile sparsity 0.8: {s * 1e3:.2f} ms "
              f"({batch / s:.0f} seq/s, {s / layers * 1e6:.0f} us/layer)")
    elif case == "bucketed":
        n_req = int(sys.argv[3]) if len(sys.argv) > 3 else 512
        d, heads, ff = 768, 12, 3072
        lens = rng.integers(16, 513, size=n_req).tolist()
        batches = scheduler.bucket_by_length(lens, max_tokens=8192, width=64, max_batch=64)
        model = make_model(et.KIND_LENGTH, layers, d, heads, ff, 0.75, 8192, 512)
        model.reserve(max(b.tokens for b in batches), 64, 512)
        xs = [torch.randn((b.tokens, d), device="cuda").half() for b in batches]
        outs = [torch.zeros_like(x) for x in xs]

        def run_all():
            for b, x, o in zip(batches, xs, outs):
                model.run_batch(o, x, b.lengths)
        s = timed(run_all, 3, warm=3)
        print(f"{layers} layers, {n_req} requests of length U[16,512] in {len(batches)} length-bucketed batches "
              f"(padding waste if padded to the bucket: {scheduler.padding_waste(batches):.1%}): {s * 1e3:.1f} ms, "
              f"{n_req / s:.0f} seq/s, {sum(lens) / s / 1e6:.2f} M tokens/s")
    elif case == "pruned":
        batch = int(sys.argv[3]) if len(sys.argv) > 3 else 32
        d, heads, ff, S = 768, 12, 3072, 256
        T = batch * S
        wrng = np.random.default_rng(0)
        ones, zeros = np.ones(d, np.float16), np.zeros(d, np.float16)

        def row_weight(ids):
            nrow = (len(ids) + 15) // 16 * 16
            w = np.zeros((nrow, d), np.float16)
            w[:len(ids)] = (wrng.standard_normal((len(ids), d), dtype=np.float32) * 0.02).astype(np.float16)
            return et.RowWeight(d, d, T, w, ids, np.zeros(nrow, np.float16), heads)
        encs = []
        for i in range(layers):
            qk_ids = et.gen_sparse_row_mat(d, 0.5, 300 + i, nhead=heads)   # Q and K keep the same dimensions
            v_ids = et.gen_sparse_row_mat(d, 0.5, 400 + i, nhead=heads)
            encs.append(et.Encoder(et.KIND_PRUNE_QKV, d, S, heads, None, row_weight(qk_ids), row_weight(qk_ids),
                                   row_weight(v_ids), tile_weight(wrng, d, d, 0.75, T, 100 * i + 3),
                                   tile_weight(wrng, d, ff, 0.75, T, 100 * i + 4, gelu=True),
                                   tile_weight(wrng, ff, d, 0.75, T, 100 * i + 5), (ones, zeros, ones, zeros)))
        model = et.Model(encs)
        x = torch.randn((T, d), device="cuda").half()
        out = torch.zeros_like(x)
        s = timed(lambda: model.run_batch(out, x, [S] * batch), 10)
        print(f"{layers} layers, Q/K/V rows pruned to half per head, {batch} x {S} tokens: {s * 1e3:.2f} ms "
              f"({batch / s:.0f} seq/s, {s / layers * 1e6:.0f} us/layer)")
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main()
