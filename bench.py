#!/usr/bin/env python
"""Benchmark of the encoder hot path on B200: one JSON line per run.

Workload: the 24-layer tile-pruned BERT-large encoder (hidden 1024, 16 heads x 64, FFN 4096, 80 % of the 16x16
weight tiles pruned by a seeded Bernoulli mask, fp16 storage, fp32 accumulate) over a batch of 256 sequences of
512 tokens. With N ranks the batch is split into N contiguous shards of 256/N sequences, one process per GPU,
no collective inside the layers; the output shards are gathered with one NCCL all-gather per step on a side
stream, joined inside the timed region (strong scaling: the total work is fixed). A step is one forward of all
24 layers over the rank's shard through et_model_run_batch (all launches replayed as one CUDA graph).

`value` is sequences per second with the inputs resident in HBM; `e2e` is the same through the public call with
pinned host buffers: every step's input crosses PCIe to the device and its result comes back inside the timed
region (copy-in, layers and copy-out pipelined on three streams). The activations of a shard (268 MB of input
at N=1, 1.3 GB of scratch) exceed the 126 MB L2, so no step finds its inputs cached.

`--impl reference` runs the reference project's own CUDA kernels (library prebuilt from the reference checkout
under oracle/_ref/) on the same workload, composed in the reference's op order, one replica per rank on that
rank's shard; where that library or a GPU is absent it times the fp32 CPU oracle on a bounded sample instead.

Both arms also report the other named configurations of the workload family under `configs` (one GPU only):
the dense single-sequence layer, the 16 x 128 tile-pruned layer at three sparsities, the attention-aware pruned
layer, and the 12-layer variable-length model against its padded form.
"""
import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "encoder sequences/sec (24-layer tile-pruned BERT-large, 256 x 512 tokens)"
LARGE = dict(d=1024, H=16, ff=4096, S=512, B=256, layers=24, sparsity=0.8)
BASE = dict(d=768, H=12, ff=3072)
LOG2E = 1.4426950408889634
# DRAM traffic of the dominant kernel from its ncu capture (profiles/): bytes per launch divided by the
# algorithmic bytes of that launch (activations once, packed weight once, output once). Used to scale the
# algorithmic bytes of the bench's launches; None where no capture exists.
NCU_TRAFFIC_RATIO = {"tile_gemm_kernel": 1.0, "source": "profiles/tile_gemm_kernel_T16384_K1024_N4096_s80.md: 35.3 MB read "
                     "= activations + packed weight; writes = the output"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the GPU is under load (only samples taken between
    mark_start() and mark_end() count)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None
        self.t0, self.t1 = None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark_start(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, s in self.samples:
            if self.t0 is not None and (t < self.t0 or (self.t1 is not None and t > self.t1 + 0.15)):
                continue
            try:
                sm.append(float(s[0])); mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ synthetic data
def layer_arrays(gen, d, ff, sparsity, seed, qk_sparsity=None):
    """Host arrays of one layer's six tile-pruned linears in the reference's format:
    name -> (row_ptr, row_offset, data[ntile, 256], bias, out_feat, in_feat). Kept tiles ~N(0, 0.02), biases 0.
    `gen(nrow, ncol, sparsity, seed, bernoulli)` is the seeded tile-pattern generator (the library's in the native
    arm, the oracle's in the reference arm; the two are bit-identical)."""
    shapes = {"q": (d, d), "k": (d, d), "v": (d, d), "o": (d, d), "ffn1": (d, ff), "ffn2": (ff, d)}
    lin = {}
    for i, (name, (K, N)) in enumerate(shapes.items()):
        s = qk_sparsity if (qk_sparsity is not None and name in "qkv") else sparsity
        rp, ro = gen(N, K, s, seed + 10 * i, True)
        data = (np.random.default_rng(seed + 10 * i + 1).standard_normal((len(ro), 256), dtype=np.float32) * 0.02).astype(np.float16)
        lin[name] = (rp, ro, data, np.zeros(N, np.float16), N, K)
    return lin


def sequence_inputs(first, count, S, d):
    """Activations ~N(0,1) of sequences first..first+count-1, each from its own seed, so that any rank can
    regenerate any shard."""
    out = np.empty((count * S, d), dtype=np.float16)
    for i in range(count):
        out[i * S:(i + 1) * S] = np.random.default_rng(100000 + first + i).standard_normal((S, d), dtype=np.float32)
    return out


def gemm_flops(lin, tokens):
    return sum(2.0 * tokens * 256 * len(v[1]) for v in lin.values())


def cfg_text(c, world):
    return (f"config 5: {c['layers']}-layer BERT-large encoder, batch {c['B']} x seq {c['S']}, hidden {c['d']}, {c['H']} heads, "
            f"FFN {c['ff']}, Bernoulli 16x16 tile sparsity {c['sparsity']}; batch split into {world} shard(s) of "
            f"{c['B'] // world} sequences")


def is_config5(c):
    return all(c[k] == LARGE[k] for k in LARGE)


# ------------------------------------------------------------------------------------------ timing helpers
def time_loop(torch, fn, n, warm, stream):
    """ms per call of fn() (which launches on `stream`), CUDA events on that stream, after `warm` untimed calls."""
    with torch.cuda.stream(stream):
        for _ in range(warm):
            fn()
        stream.synchronize()
        if n <= 0:
            return 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) / n


def reps_for(ms_per_step, steps, min_seconds=0.5, cap=25):
    return int(max(1, min(cap, math.ceil(min_seconds / max(1e-6, ms_per_step * 1e-3 * steps)))))


# ------------------------------------------------------------------------------------------ CPU baseline
def cpu_baseline(orc, c):
    """The fp32 oracle (a CPU port of the layer) on the host cores, on a bounded sample of the workload: one of the
    identical-shape layers over a few of the sequences, scaled to whole sequences through all layers."""
    nseq = 4
    lin = layer_arrays(orc.gen_sparse_tile_mat, c["d"], c["ff"], c["sparsity"], 1000)
    ol = {k: v[:5] for k, v in lin.items()}
    ln = ((np.ones(c["d"], np.float16), np.zeros(c["d"], np.float16)),) * 2
    X = sequence_inputs(0, nseq, c["S"], c["d"])
    reps, t0 = 0, time.perf_counter()
    while True:
        orc.encoder_layer(X, ol, ln, [c["S"]] * nseq, c["d"], c["H"])
        reps += 1
        el = time.perf_counter() - t0
        if el > 10.0 or reps >= 50:
            break
    per_layer_seq = el / (reps * nseq)
    return {"value": 1.0 / (per_layer_seq * c["layers"]), "unit": "sequences/s", "cores": orc.threads(), "kind": "port",
            "sample": f"{reps} forwards of ONE layer over {nseq} sequences of {c['S']} tokens ({el:.1f} s of CPU work), scaled "
                      f"linearly to {c['layers']} layers; fp32 oracle with OpenMP"}


# ------------------------------------------------------------------------------------------ reference arm
class Bsr(ctypes.Structure):
    _fields_ = [("row_ptr", ctypes.c_void_p), ("row_offset", ctypes.c_void_p), ("data", ctypes.c_void_p),
                ("bias", ctypes.c_void_p)]


def run_reference(args, c, rank, world, local_rank):
    """Reference arm: the reference's own CUDA kernels, one replica per rank on that rank's shard, or the CPU oracle
    where they cannot run."""
    from tests import oracle_lib
    orc = oracle_lib.load()
    base = {"metric": METRIC, "unit": "sequences/s", "impl": "reference", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": {"workload": cfg_text(c, world), "global_batch": c["B"], "seq_len": c["S"],
                                            "sparsity": c["sparsity"], "parallelism": f"dp{world}" if world > 1 else "single"}}
    ref = oracle_lib.load_ref()
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if ref is None or not have_gpu:
        if rank != 0:
            return
        cpu = cpu_baseline(orc, c)
        base.update({"value": cpu["value"], "ms_per_step": 1e3 * c["B"] / cpu["value"], "cpu_baseline": cpu,
                     "reference_kind": "fp32 CPU oracle (the reference ships no CPU path; its CUDA library or a GPU is absent here)",
                     "e2e": {"value": cpu["value"], "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        print(json.dumps(base))
        return
    import torch
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    vp = ctypes.c_void_p
    stream = torch.cuda.Stream()
    sp = vp(stream.cuda_stream)

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    class RefLayer:
        def __init__(self, lin, d):
            self.keep, self.arr = [], (Bsr * 6)()
            for i, name in enumerate(["q", "k", "v", "o", "ffn1", "ffn2"]):
                ts = [dev(a) for a in lin[name][:4]]
                self.keep.append(ts)
                self.arr[i] = Bsr(*[t.data_ptr() for t in ts])
            self.ln = [torch.ones(d, dtype=torch.float16, device="cuda"), torch.zeros(d, dtype=torch.float16, device="cuda")]

    def tile_stack(cfg, n_layers, seq, batch, seed0):
        """step(x, y): n_layers of the reference's tile layer over batch x seq tokens, y <- layers(x)."""
        d, H, ff = cfg["d"], cfg["H"], cfg["ff"]
        layers = [RefLayer(layer_arrays(orc.gen_sparse_tile_mat, d, ff, cfg["sparsity"], seed0 + 1000 * l), d) for l in range(n_layers)]
        T = seq * batch
        buf = torch.zeros(8 * T * d, dtype=torch.float16, device="cuda")
        mask = torch.zeros((seq, seq), dtype=torch.float16, device="cuda")
        scale = ctypes.c_float(LOG2E / (d // H) ** 0.5)   # the kernel exponentiates in base 2: this gives the true softmax

        def step(x, y):
            for l, L in enumerate(layers):
                src = x if l == 0 else y
                rc = ref.ref_encoder_tile_layer(vp(y.data_ptr()), vp(src.data_ptr()), vp(buf.data_ptr()), L.arr,
                                                vp(L.ln[0].data_ptr()), vp(L.ln[1].data_ptr()), vp(L.ln[0].data_ptr()),
                                                vp(L.ln[1].data_ptr()), vp(mask.data_ptr()), batch, seq, d, H, ff, scale, sp)
                assert rc == 0, "reference tile layer failed"
        step.keep = (layers, buf, mask)
        return step

    Br = c["B"] // world
    T = Br * c["S"]
    step = tile_stack(c, c["layers"], c["S"], Br, 1000)
    X = sequence_inputs(rank * Br, Br, c["S"], c["d"])
    x = dev(X)
    y = torch.zeros_like(x)
    with ClockSampler(local_rank) as cs:
        est = time_loop(torch, lambda: step(x, y), 1, 1, stream)
        R = reps_for(est, args.steps)
        time_loop(torch, lambda: step(x, y), 0, max(0, args.warmup - 1), stream)
        cs.mark_start()
        times = []
        for _ in range(R):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ms = time_loop(torch, lambda: step(x, y), args.steps, 0, stream)
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
            times.append(ms)
        cs.mark_end()
    ms = statistics.median(times)
    # end to end: the shard's input from pinned host memory, all layers, the result back, one step at a time
    hx = torch.from_numpy(X).pin_memory()
    ho = torch.empty_like(hx).pin_memory()
    n_e2e = max(2, min(args.steps, 5))

    def e2e_step():
        with torch.cuda.stream(stream):
            x.copy_(hx, non_blocking=True)
            step(x, y)
            ho.copy_(y, non_blocking=True)
        stream.synchronize()
    e2e_step()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_s = (time.perf_counter() - t0) / n_e2e
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = t.item()
    value = c["B"] / (ms * 1e-3)
    base.update({"value": value, "ms_per_step": ms, "us_per_layer": ms * 1e3 / c["layers"], "timed_repetitions": R,
                 "ms_per_step_all_repetitions": times, "clocks": cs.summary(),
                 "reference_kind": "the reference's own CUDA kernels (oracle/_ref), one replica per rank on that rank's shard: "
                                   "per layer the six tile linears and both LayerNorms once over all tokens, its on-the-fly "
                                   "attention kernel once per sequence, one stream, no host synchronisation",
                 "cpu_baseline": {"value": value, "unit": "sequences/s", "cores": 0, "kind": "reference",
                                  "sample": "not a CPU figure: the reference has no CPU implementation, this arm runs its CUDA "
                                            "kernels on the same GPU(s) over the full workload"},
                 "e2e": {"value": c["B"] / e2e_s, "unit": "sequences/s", "h2d_bytes_per_step": int(hx.numel() * 2),
                         "d2h_bytes_per_step": int(ho.numel() * 2), "steps": n_e2e,
                         "how": "per step: shard input host to device, all layers, result device to host, then a host "
                                "synchronisation (bytes per rank)"}})
    del step, x, y, hx, ho
    if rank == 0 and world == 1 and not args.no_extras:
        base["configs"] = reference_configs(torch, ref, orc, tile_stack, stream, dev)
        base["configs"]["c5"] = {"sequences_per_s": value, "us_per_layer": ms * 1e3 / c["layers"]}
    if rank == 0:
        print(json.dumps(base))
    if world > 1:
        dist.destroy_process_group()


def reference_configs(torch, ref, orc, tile_stack, stream, dev):
    """The reference's kernels on the other named configurations (one GPU)."""
    vp = ctypes.c_void_p
    sp = vp(stream.cuda_stream)
    out = {}
    d, H, ff = BASE["d"], BASE["H"], BASE["ff"]

    def run_tile(B, S, sparsity, n=200):
        cfg = dict(BASE, sparsity=sparsity)
        insts = max(2, min(12, int(-(-300e6 // (7 * B * S * d * 2 + 14.2e6 * (1 - sparsity))))))
        steps = [tile_stack(cfg, 1, S, B, 7000 + 17 * i) for i in range(insts)]
        xs = [dev(sequence_inputs(1000 * i, B, S, d)) for i in range(insts)]
        ys = [torch.zeros_like(t) for t in xs]
        k = [0]

        def fn():
            i = k[0] % insts
            k[0] += 1
            steps[i](xs[i], ys[i])
        ms = time_loop(torch, fn, n, 2 * insts, stream)
        return {"us_per_layer": ms * 1e3, "sequences_per_s": B / (ms * 1e-3), "instances_rotated": insts}
    out["c1"] = dict(run_tile(1, 128, 0.0), what="dense base layer, 1 x 128 tokens")
    out["c2"] = {str(s): run_tile(16, 128, s) for s in (0.5, 0.75, 0.9)}
    out["c2"]["what"] = "tile-pruned base layer, 16 x 128 tokens, one batch at a time"

    # c3: Q and K tile-pruned at 50 % (the reference cannot row-prune them), V row-pruned to half of every head,
    # output projection and FFN tile-pruned at 75 %; its pruned-attention kernel as shipped (stores nothing).
    B, S = 32, 256
    T = B * S
    lin = layer_arrays(orc.gen_sparse_tile_mat, d, ff, 0.75, 7100, qk_sparsity=0.5)
    keep, arr = [], (Bsr * 6)()
    for i, name in enumerate(["q", "k", "v", "o", "ffn1", "ffn2"]):
        ts = [dev(a) for a in lin[name][:4]]
        keep.append(ts)
        arr[i] = Bsr(*[t.data_ptr() for t in ts])
    ids = orc.gen_sparse_row_mat(d, 0.5, 7200, nhead=H)
    nnz = (len(ids) + 15) // 16 * 16
    vw = np.zeros((nnz, d), np.float16)
    vw[:len(ids)] = (np.random.default_rng(7201).standard_normal((len(ids), d), dtype=np.float32) * 0.02).astype(np.float16)
    hp = orc.head_ptr(ids, H, d)
    hp[-1] = len(ids)
    vwd, vbd, idd, hpd = dev(vw), dev(np.zeros(nnz, np.float16)), dev(ids.astype(np.int32)), dev(hp.astype(np.int32))
    g, b_ = torch.ones(d, dtype=torch.float16, device="cuda"), torch.zeros(d, dtype=torch.float16, device="cuda")
    mask = torch.zeros((S, S), dtype=torch.float16, device="cuda")
    insts = 3
    xs = [dev(sequence_inputs(5000 + 100 * i, B, S, d)) for i in range(insts)]
    ys = [torch.zeros_like(t) for t in xs]
    bufs = [torch.zeros(8 * T * d, dtype=torch.float16, device="cuda") for _ in range(insts)]
    k = [0]

    def prune_fn():
        i = k[0] % insts
        k[0] += 1
        rc = ref.ref_encoder_prune_layer(vp(ys[i].data_ptr()), vp(xs[i].data_ptr()), vp(bufs[i].data_ptr()), arr, vp(vwd.data_ptr()),
                                         vp(vbd.data_ptr()), vp(idd.data_ptr()), vp(hpd.data_ptr()), nnz, vp(g.data_ptr()),
                                         vp(b_.data_ptr()), vp(g.data_ptr()), vp(b_.data_ptr()), vp(mask.data_ptr()), B, S, d, H, ff, sp)
        assert rc == 0, "reference prune layer failed"
    ms = time_loop(torch, prune_fn, 60, 6, stream)
    out["c3"] = {"us_per_layer": ms * 1e3, "sequences_per_s": B / (ms * 1e-3), "instances_rotated": insts,
                 "what": "32 x 256 tokens; Q/K tile-pruned 50 % (the reference's Encoder_prune row-prunes V only), V row-pruned "
                         "50 %, output projection and FFN tile-pruned 75 %; its pruned-attention kernel as shipped computes "
                         "the attention and never stores it, which only shortens its time"}
    xr = [dev(sequence_inputs(6000 + 100 * i, B, S, d)) for i in range(8)]
    wr = [dev((np.random.default_rng(7290 + i).standard_normal((nnz, d), dtype=np.float32) * 0.02).astype(np.float16)) for i in range(8)]
    yr = [torch.zeros((T, nnz), dtype=torch.float16, device="cuda") for _ in range(8)]
    k[0] = 0

    def row_fn():
        i = k[0] % 8
        k[0] += 1
        rc = ref.ref_row_spmm(vp(yr[i].data_ptr()), vp(xr[i].data_ptr()), vp(wr[i].data_ptr()), vp(vbd.data_ptr()), T, nnz, d, sp)
        assert rc == 0, "reference row linear failed"
    ms_r = time_loop(torch, row_fn, 200, 16, stream)
    out["c3_row_linear"] = {"us": ms_r * 1e3, "tflops": 2.0 * T * len(ids) * d / (ms_r * 1e-3) / 1e12,
                            "what": f"the reference's row-pruned launcher alone (bias fill + cuBLAS GEMM), {T} tokens, {len(ids)} of {d} "
                                    "output features kept, eight weight/activation sets rotated"}
    del xs, ys, bufs, xr, wr, yr

    # c4: 12 layers, 64 sequences with lengths U[32,512] rounded UP to 16 (the reference's kernels need multiples of
    # 16), scores GEMM + shared-QK attention per sequence; against the same batch padded to 512.
    lens = np.random.default_rng(4242).integers(32, 513, size=64)
    lens16 = ((lens + 15) // 16 * 16).astype(np.int32)
    cfg = dict(BASE, sparsity=0.75)
    layers = []
    for l in range(12):
        ll = layer_arrays(orc.gen_sparse_tile_mat, d, ff, 0.75, 7300 + 1000 * l)
        kp, ar = [], (Bsr * 6)()
        for i, name in enumerate(["q", "k", "v", "o", "ffn1", "ffn2"]):
            ts = [dev(a) for a in ll[name][:4]]
            kp.append(ts)
            ar[i] = Bsr(*[t.data_ptr() for t in ts])
        layers.append((kp, ar))
    scores = torch.zeros(H * 512 * 512, dtype=torch.float16, device="cuda")
    mask = torch.zeros((512, 512), dtype=torch.float16, device="cuda")

    def length_model(lens_arr):
        Tt = int(lens_arr.sum())
        x = torch.randn((Tt, d), device="cuda").half()
        y = torch.zeros_like(x)
        buf = torch.zeros(8 * Tt * d, dtype=torch.float16, device="cuda")
        la = np.ascontiguousarray(lens_arr, dtype=np.int32)

        def fn():
            for l, (kp, ar) in enumerate(layers):
                src = x if l == 0 else y
                rc = ref.ref_encoder_length_layer(vp(y.data_ptr()), vp(src.data_ptr()), vp(buf.data_ptr()), vp(scores.data_ptr()), ar,
                                                  vp(g.data_ptr()), vp(b_.data_ptr()), vp(g.data_ptr()), vp(b_.data_ptr()),
                                                  vp(mask.data_ptr()), vp(la.ctypes.data), len(la), d, H, ff, sp)
                assert rc == 0, "reference length layer failed"
        ms_ = time_loop(torch, fn, 5, 2, stream)
        return ms_, Tt
    ms_p, Tp = length_model(lens16)
    ms_f, Tf = length_model(np.full(64, 512, dtype=np.int32))
    out["c4"] = {"ms_per_model_packed": ms_p, "sequences_per_s_packed": 64 / (ms_p * 1e-3), "tokens_packed": Tp,
                 "ms_per_model_padded_512": ms_f, "sequences_per_s_padded_512": 64 / (ms_f * 1e-3), "tokens_padded": Tf,
                 "what": "12 base layers, 64 sequences of length U[32,512] rounded up to 16, tile sparsity 0.75: scores GEMM "
                         "(cuBLAS, strided over the heads) into HBM and the shared-QK attention kernel once per sequence, zero mask"}
    return out


# ------------------------------------------------------------------------------------------ native arm
def build_model(et, c, tokens, kind=None, seq=None, n_layers=None, seed0=1000):
    ones, zeros = np.ones(c["d"], np.float16), np.zeros(c["d"], np.float16)
    encs, first_lin = [], None
    for l in range(c["layers"] if n_layers is None else n_layers):
        lin = layer_arrays(et.gen_sparse_tile_mat, c["d"], c["ff"], c["sparsity"], seed0 + 1000 * l)
        if first_lin is None:
            first_lin = lin
        w = {n: et.TileWeight(v[5], v[4], tokens, v[2], v[0], v[1], v[3], is_gelu=(n == "ffn1")) for n, v in lin.items()}
        encs.append(et.Encoder(et.KIND_TILE if kind is None else kind, c["d"], c["S"] if seq is None else seq, c["H"], None,
                               w["q"], w["k"], w["v"], w["o"], w["ffn1"], w["ffn2"], (ones, zeros, ones, zeros)))
    return et.Model(encs), first_lin


def native_configs(torch, et, stream, pk):
    """The other named configurations on one GPU through the same public objects."""
    out = {}
    d, H, ff = BASE["d"], BASE["H"], BASE["ff"]

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def run_tile(B, S, sparsity, n=300, streams=1):
        cfg = dict(BASE, sparsity=sparsity, S=S, layers=1)
        T = B * S
        insts = max(2, min(12, int(-(-300e6 // (7 * T * d * 2 + 14.2e6 * (1 - sparsity))))))
        if streams > 1:
            insts = 12
        models = [build_model(et, cfg, T, n_layers=1, seed0=7000 + 17 * i)[0] for i in range(insts)]
        xs = [dev(sequence_inputs(1000 * i, B, S, d)) for i in range(insts)]
        ys = [torch.zeros_like(t) for t in xs]
        lens = [S] * B
        k = [0]
        if streams == 1:
            def fn():
                i = k[0] % insts
                k[0] += 1
                models[i].run_batch(ys[i], xs[i], lens, stream=stream)
            ms = time_loop(torch, fn, n, 3 * insts, stream)
        else:
            side = [torch.cuda.Stream() for _ in range(streams)]

            def fn_all():   # one round over all instances, instance i always on stream i mod streams
                for s_ in side:
                    s_.wait_stream(stream)
                for i in range(insts):
                    models[i].run_batch(ys[i], xs[i], lens, stream=side[i % streams])
                for s_ in side:
                    stream.wait_stream(s_)
            ms = time_loop(torch, fn_all, max(1, n // insts), 3, stream) / insts
        for m in models:
            m.check()
        return {"us_per_layer": ms * 1e3, "sequences_per_s": B / (ms * 1e-3), "instances_rotated": insts}
    out["c1"] = dict(run_tile(1, 128, 0.0), what="dense base layer, 1 x 128 tokens")
    out["c2"] = {str(s): run_tile(16, 128, s) for s in (0.5, 0.75, 0.9)}
    out["c2"]["what"] = "tile-pruned base layer, 16 x 128 tokens, one batch at a time, weights packed for the shortest launch"
    et.set_tuning_goal("throughput")
    try:
        r = run_tile(16, 128, 0.75, n=1200, streams=6)
    finally:
        et.set_tuning_goal("latency")
    out["c2"]["0.75_six_batches_in_flight"] = dict(r, what="six independent batches in flight on six streams, weights packed for "
                                                             "the least SM time per launch; us_per_layer is time per batch")

    # c3: Q, K and V row-pruned to half of every head (Q and K keep the same dimensions), output projection and FFN
    # tile-pruned at 75 %
    B, S = 32, 256
    T = B * S
    ones, zeros = np.ones(d, np.float16), np.zeros(d, np.float16)
    wrng = np.random.default_rng(7201)

    def row_weight(ids):
        nrow = (len(ids) + 15) // 16 * 16
        w = np.zeros((nrow, d), np.float16)
        w[:len(ids)] = (wrng.standard_normal((len(ids), d), dtype=np.float32) * 0.02).astype(np.float16)
        return et.RowWeight(d, d, T, w, ids, np.zeros(nrow, np.float16), H)
    insts = 3
    models = []
    for i in range(insts):
        lin = layer_arrays(et.gen_sparse_tile_mat, d, ff, 0.75, 7100 + 100 * i)
        tw = {n: et.TileWeight(v[5], v[4], T, v[2], v[0], v[1], v[3], is_gelu=(n == "ffn1")) for n, v in lin.items() if n in ("o", "ffn1", "ffn2")}
        qk_ids = et.gen_sparse_row_mat(d, 0.5, 7200 + i, nhead=H)
        v_ids = et.gen_sparse_row_mat(d, 0.5, 7250 + i, nhead=H)
        models.append(et.Model([et.Encoder(et.KIND_PRUNE_QKV, d, S, H, None, row_weight(qk_ids), row_weight(qk_ids), row_weight(v_ids),
                                           tw["o"], tw["ffn1"], tw["ffn2"], (ones, zeros, ones, zeros))]))
    xs = [dev(sequence_inputs(5000 + 100 * i, B, S, d)) for i in range(insts)]
    ys = [torch.zeros_like(t) for t in xs]
    k = [0]

    def prune_fn():
        i = k[0] % insts
        k[0] += 1
        models[i].run_batch(ys[i], xs[i], [S] * B, stream=stream)
    ms = time_loop(torch, prune_fn, 90, 9, stream)
    out["c3"] = {"us_per_layer": ms * 1e3, "sequences_per_s": B / (ms * 1e-3), "instances_rotated": insts,
                 "what": "32 x 256 tokens; Q, K and V row-pruned to half of every head, output projection and FFN tile-pruned 75 %"}
    # the row-pruned linear alone at this shape (the reference runs cuBLAS there)
    rws = [row_weight(et.gen_sparse_row_mat(d, 0.5, 7290 + i, nhead=H)) for i in range(8)]
    yr = [torch.zeros((T, rws[0].nrow), dtype=torch.float16, device="cuda") for _ in range(8)]
    xr = [dev(sequence_inputs(6000 + 100 * i, B, S, d)) for i in range(8)]
    k[0] = 0

    def row_fn():
        i = k[0] % 8
        k[0] += 1
        rws[i].run(yr[i], xr[i], stream=stream)
    ms_r = time_loop(torch, row_fn, 200, 16, stream)
    out["c3_row_linear"] = {"us": ms_r * 1e3, "tflops": 2.0 * T * rws[0].row_id_size * d / (ms_r * 1e-3) / 1e12,
                            "what": f"row-pruned linear alone, {T} tokens, {rws[0].row_id_size} of {d} output features kept, in_feat {d}, "
                                    "eight weight/activation sets rotated"}
    del models, xs, ys, rws, yr, xr

    # c4: 12 layers, 64 sequences of length U[32,512], packed (length-driven tiling) against padded to 512
    lens = np.random.default_rng(4242).integers(32, 513, size=64).tolist()
    cfg = dict(BASE, sparsity=0.75, S=512, layers=12)
    Tp, Tf = sum(lens), 512 * 64
    model, _ = build_model(et, cfg, Tf, kind=et.KIND_LENGTH, seed0=7300)
    x = torch.randn((Tp, d), device="cuda").half()
    y = torch.zeros_like(x)
    ms_p = time_loop(torch, lambda: model.run_batch(y, x, lens, stream=stream), 10, 3, stream)
    xf = torch.randn((Tf, d), device="cuda").half()
    yf = torch.zeros_like(xf)
    ms_f = time_loop(torch, lambda: model.run_batch(yf, xf, [512] * 64, valid_lens=lens, stream=stream), 10, 3, stream)
    model.check()
    out["c4"] = {"ms_per_model_packed": ms_p, "sequences_per_s_packed": 64 / (ms_p * 1e-3), "tokens_packed": Tp,
                 "ms_per_model_padded_512": ms_f, "sequences_per_s_padded_512": 64 / (ms_f * 1e-3), "tokens_padded": Tf,
                 "what": "12 base layers, 64 sequences of length U[32,512] (any length, no rounding), tile sparsity 0.75; padded "
                         "form: every sequence in 512 rows with key padding"}
    del model, x, y, xf, yf

    # bandwidth kernels on inputs larger than L2
    rows, dm = 131072, 1024
    a = torch.randn((rows, dm), device="cuda").half(); b = torch.randn((rows, dm), device="cuda").half()
    g = torch.ones(dm, dtype=torch.float16, device="cuda"); be = torch.zeros(dm, dtype=torch.float16, device="cuda")
    ln_ms = time_loop(torch, lambda: et.skip_layernorm(a, b, g, be, stream=stream), 20, 3, stream)
    gbs = 6.0 * dm * rows / (ln_ms * 1e-3) / 1e9
    out["roofline_layernorm"] = {"kernel": "skip_layernorm_vec", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / pk["hbm_gbs"], "rows": rows, "size": dm, "bytes_per_row": 6 * dm}
    del a, b
    nmat, L = 16 * 64, 512
    Sm = torch.randn((nmat, L, L), device="cuda").half()
    sm_ms = time_loop(torch, lambda: et.softmax_mask(Sm, stream=stream), 20, 3, stream)
    gbs = 4.0 * L * L * nmat / (sm_ms * 1e-3) / 1e9
    out["roofline_softmax"] = {"kernel": "softmax_mask_vec", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                               "frac": gbs / pk["hbm_gbs"], "matrices": nmat, "seq_len": L, "bytes_per_matrix": 4 * L * L}
    del Sm
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--layers", type=int, default=LARGE["layers"], help="debugging only: anything but 24 is not the named workload")
    ap.add_argument("--batch", type=int, default=LARGE["B"], help="debugging only: global batch (256 is the named workload)")
    ap.add_argument("--seq", type=int, default=LARGE["S"], help="debugging only")
    ap.add_argument("--ln-fusion", action="store_true", help="debugging only: the layer stack's optional form with the LayerNorms folded "
                    "into the linears (5 launches per layer instead of 7; slower on B200, off by default in the library)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations and the bandwidth legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    c = dict(LARGE, layers=args.layers, B=args.batch, S=args.seq)
    if c["B"] % world:
        raise SystemExit(f"the batch of {c['B']} sequences does not split into {world} equal shards")
    if args.impl == "reference":
        run_reference(args, c, rank, world, local_rank)
        return

    import torch
    import et_b200 as et
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    et.lib()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pk = peaks()
    Br = c["B"] // world
    T = Br * c["S"]
    d = c["d"]
    lens = [c["S"]] * Br
    comp, gstream, s_in, s_out = (torch.cuda.Stream() for _ in range(4))

    with ClockSampler(local_rank) as cs:
        model, lin0 = build_model(et, c, T)
        if args.ln_fusion:
            model.set_layernorm_fusion(True)
        fused = model.layernorm_fused
        launches_per_layer = 5 if fused else 7
        model.reserve(T, Br, c["S"])
        X = sequence_inputs(rank * Br, Br, c["S"], d)
        x = torch.from_numpy(X).cuda()
        outs = [torch.zeros_like(x) for _ in range(2)]
        gathered = [torch.zeros((world * T, d), dtype=torch.float16, device="cuda") for _ in range(2)] if world > 1 else None
        ev_done = [torch.cuda.Event() for _ in range(2)]     # step finished writing outs[k]
        ev_gathered = [torch.cuda.Event() for _ in range(2)]  # the all-gather that read outs[k] has completed
        count = [0]

        def step():
            i = count[0]
            k = i % 2
            count[0] += 1
            if world > 1 and i >= 2:
                comp.wait_event(ev_gathered[k])       # outs[k] is written again only after its gather has read it
            model.run_batch(outs[k], x, lens, stream=comp)
            if world > 1:
                ev_done[k].record(comp)
                with torch.cuda.stream(gstream):
                    gstream.wait_event(ev_done[k])
                    dist.all_gather_into_tensor(gathered[k], outs[k])
                    ev_gathered[k].record(gstream)

        def run_steps(n):
            """ms per step over exactly n steps, device time on the compute stream, gathers joined before the closing event."""
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(comp):
                e0.record(comp)
                for _ in range(n):
                    step()
                if world > 1:
                    comp.wait_stream(gstream)
                e1.record(comp)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ms_ = e0.elapsed_time(e1) / n
            if world > 1:
                t = torch.tensor([ms_], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_ = t.item()
            return ms_

        run_steps(6)              # direct run, graph capture and first replay on both output buffers
        est = run_steps(args.warmup)
        R = reps_for(est, args.steps)
        if world > 1:             # every rank must time the same number of repetitions
            t = torch.tensor([R], dtype=torch.int64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            R = int(t.item())
        cs.mark_start()
        times = [run_steps(args.steps) for _ in range(R)]
        cs.mark_end()
    ms = statistics.median(times)
    clocks = cs.summary()
    value = c["B"] / (ms * 1e-3)
    model.check()   # raises if a bounded device-side wait gave up during the timed region

    # ---- the gathered output against the ranks' own results
    gather_check = None
    if world > 1:
        run_steps(2)
        k = (count[0] - 1) % 2
        own = bool(torch.equal(gathered[k][rank * T:(rank + 1) * T], outs[k]))
        peer = (rank + 1) % world
        xp = torch.from_numpy(sequence_inputs(peer * Br, Br, c["S"], d)).cuda()
        yp = torch.zeros_like(xp)
        model.run_batch(yp, xp, lens, stream=comp)
        comp.synchronize()
        same = bool(torch.equal(gathered[k][peer * T:(peer + 1) * T], yp))
        flags = torch.tensor([int(own), int(same)], dtype=torch.int64, device="cuda")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        gather_check = {"own_shard_in_gathered_output_bit_equal": bool(flags[0].item()),
                        "neighbour_shard_recomputed_here_bit_equal": bool(flags[1].item()),
                        "what": "after the timed region: every rank compares its slice of the gathered output with its own "
                                "result, and recomputes the next rank's shard from that shard's seeded input on its own GPU "
                                "and compares it with the gathered slice (minimum over ranks)"}
        del xp, yp

    # ---- end to end through the public call with host buffers
    hx = torch.from_numpy(X).pin_memory()
    full = world > 1 and rank == 0
    ho = [torch.empty((world * T if full else T, d), dtype=torch.float16).pin_memory() for _ in range(2)]
    xin = [torch.zeros_like(x) for _ in range(2)]
    ev_in, ev_comp, ev_g, ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(4))
    used = [False, False]
    n_e2e = max(3, min(args.steps, 10))

    def e2e_step(i):
        k = i % 2
        if used[k]:
            ev_out[k].synchronize()           # the host has the result of the step that used this buffer set
        with torch.cuda.stream(s_in):
            xin[k].copy_(hx, non_blocking=True)
            ev_in[k].record(s_in)
        with torch.cuda.stream(comp):
            comp.wait_event(ev_in[k])
            model.run_batch(outs[k], xin[k], lens, stream=comp)
            ev_comp[k].record(comp)
        src, last = outs[k], ev_comp[k]
        if world > 1:
            with torch.cuda.stream(gstream):
                gstream.wait_event(ev_comp[k])
                dist.all_gather_into_tensor(gathered[k], outs[k])
                ev_g[k].record(gstream)
            last = ev_g[k]
            if full:
                src = gathered[k]
        with torch.cuda.stream(s_out):
            s_out.wait_event(last)
            ho[k].copy_(src, non_blocking=True)
            ev_out[k].record(s_out)
        used[k] = True
    for i in range(6):
        e2e_step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / n_e2e
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = t.item()
    e2e = {"value": c["B"] / e2e_s, "unit": "sequences/s", "h2d_bytes_per_step": int(hx.numel() * 2),
           "d2h_bytes_per_step": int(ho[0].numel() * 2), "steps": n_e2e,
           "how": "per step and rank: the shard's input from pinned host memory to the device, all layers through "
                  "et_model_run_batch, the result back to pinned host memory (rank 0 of a multi-GPU run copies the whole "
                  "gathered output, the other ranks their own shard); copy-in, layers and copy-out of consecutive steps "
                  "overlap on three streams over two buffer sets; wall clock, maximum over ranks"}
    del hx, ho, xin

    # ---- roofline of the dominant kernel: the four tile-GEMM launches of one layer at the shard's token count,
    # each timed alone with CUDA events on its stream (operands far larger than L2)
    qkv_rp = np.concatenate([lin0["q"][0], lin0["k"][0][1:] + lin0["q"][0][-1],
                             lin0["v"][0][1:] + lin0["q"][0][-1] + lin0["k"][0][-1]]).astype(np.int32)
    wq = et.TileWeight(d, 3 * d, T, np.concatenate([lin0[n][2] for n in "qkv"]), qkv_rp,
                       np.concatenate([lin0[n][1] for n in "qkv"]), np.concatenate([lin0[n][3] for n in "qkv"]))
    wo, w1, w2 = (et.TileWeight(lin0[n][5], lin0[n][4], T, lin0[n][2], lin0[n][0], lin0[n][1], lin0[n][3]) for n in ("o", "ffn1", "ffn2"))
    hbuf = torch.randn((T, c["ff"]), device="cuda").half()
    ybuf = torch.zeros((T, c["ff"]), dtype=torch.float16, device="cuda")
    launches = [("fused Q|K|V", wq, ybuf, x, False), ("output projection", wo, ybuf, x, False),
                ("FFN1 + GELU", w1, ybuf, x, True), ("FFN2", w2, outs[0], hbuf, False)]
    per, tot_ms, tot_fl, tot_bytes = [], 0.0, 0.0, 0.0
    for name, w, yb, xb, gelu in launches:
        ms_l = time_loop(torch, lambda: w.run(yb, xb, gelu=gelu, stream=comp), 10, 3, comp)
        fl = 2.0 * T * 256 * w.ntile
        alg_bytes = 2.0 * T * w.in_feat + 528.0 * w.ntile + 2.0 * T * w.out_feat
        per.append({"launch": name, "K": w.in_feat, "N": w.out_feat, "kept_tiles": w.ntile, "ms": ms_l, "tflops": fl / (ms_l * 1e-3) / 1e12,
                    "algorithmic_bytes": alg_bytes, "packing": w.info()})
        w.check()
        tot_ms += ms_l; tot_fl += fl; tot_bytes += alg_bytes
    achieved = tot_fl / (tot_ms * 1e-3) / 1e12
    ratio = NCU_TRAFFIC_RATIO.get("tile_gemm_kernel")
    roofline = {"kernel": "tile_gemm_kernel (the 4 launches of a layer: fused Q|K|V, output, FFN1+GELU, FFN2)", "bound": "tensor",
                "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                "peak_source": pk["source"] + " (bf16 burst; each launch is timed alone)",
                "frac_of_sustained_peak": achieved / pk["tflops_sustained"] if pk.get("tflops_sustained") else None,
                "flops_per_launch_set": tot_fl, "ms_per_launch_set": tot_ms, "launches": per, "tokens": T,
                "traffic": None if ratio is None else ratio * tot_bytes,
                "traffic_note": "DRAM bytes per launch set: algorithmic bytes of these launches times the measured/algorithmic ratio "
                                "of the ncu capture of the same kernel on a smaller case (" + NCU_TRAFFIC_RATIO["source"] + ")",
                "dense_equivalent_tflops": achieved / max(1e-9, 1.0 - c["sparsity"]),
                "note": "algorithmic FLOPs count kept tiles only (2 * tokens * 256 * kept tiles)"}
    # the attention kernel alone at the same shape (tensor bound)
    qkvb = torch.randn((T, 3 * d), device="cuda").half()
    zb = torch.zeros((T, d), dtype=torch.float16, device="cuda")
    at_ms = time_loop(torch, lambda: et.attention_batch(zb, qkvb[:, :d], qkvb[:, d:2 * d], qkvb[:, 2 * d:], d, c["H"], batch=Br,
                                                        uniform_len=c["S"], max_seq_len=c["S"], qk_pitch=3 * d, v_pitch=3 * d,
                                                        stream=comp), 10, 3, comp)
    et.attention_check()
    at_fl = 4.0 * c["S"] * c["S"] * d * Br
    roofline_attention = {"kernel": "attention_tc_kernel", "bound": "tensor", "achieved": at_fl / (at_ms * 1e-3) / 1e12,
                          "peak": pk["tflops"], "unit": "TFLOP/s", "frac": at_fl / (at_ms * 1e-3) / 1e12 / pk["tflops"], "ms": at_ms,
                          "sequences": Br, "seq_len": c["S"]}
    del hbuf, ybuf, qkvb, zb

    layer_fl = gemm_flops(lin0, T) + 4.0 * c["S"] * c["S"] * d * Br
    workload = cfg_text(c, world) if is_config5(c) else "NOT the named workload (debugging flags): " + cfg_text(c, world)
    result = {"metric": METRIC, "value": value, "unit": "sequences/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
              "ms_per_step": ms, "us_per_layer": ms * 1e3 / c["layers"], "timed_repetitions": R, "ms_per_step_all_repetitions": times,
              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
              "config": {"workload": workload, "global_batch": c["B"], "seq_len": c["S"], "sparsity": c["sparsity"],
                         "parallelism": f"dp{world}" if world > 1 else "single",
                         "gather": ("one NCCL all-gather of the output shards per step on a side stream, overlapping the next step, "
                                    "joined before the closing event") if world > 1 else "none",
                         "timing": f"{R} repetition(s) of exactly {args.steps} steps, each between barrier + synchronise, CUDA events, "
                                   "maximum over ranks; the median repetition is reported",
                         "l2": "inputs larger than L2: the shard's activations (input, scratch of five token x hidden buffers, output) "
                               "are several times the 126 MB L2 and every layer streams them"},
              "clocks": clocks, "e2e": e2e, "gpu_launches": (launches_per_layer * c["layers"] + (1 if fused else 0)) * args.steps * R,
              "launches_per_step": (f"{5 * c['layers'] + 1}: per layer fused Q|K|V tile GEMM, attention, output tile GEMM (+ residual, row sums), "
                                    "FFN1 tile GEMM (normalises its input, GELU), FFN2 tile GEMM (+ LayerNorm of the residual, row sums); one "
                                    "LayerNorm at the end; all replayed as one CUDA graph") if fused else
                                   (f"{7 * c['layers']}: per layer fused Q|K|V tile GEMM, attention, output tile GEMM, LayerNorm, FFN1 tile "
                                    "GEMM (GELU), FFN2 tile GEMM, LayerNorm; all layers replayed as one CUDA graph"),
              "layernorm_folded_into_linears": fused,
              "roofline": roofline, "roofline_attention": roofline_attention,
              "model_tflops": layer_fl * c["layers"] * world / (ms * 1e-3) / 1e12, "gather_check": gather_check,
              "device_error_words": 0}
    del model, x, outs
    if rank == 0 and world == 1 and not args.no_extras:
        extras = native_configs(torch, et, comp, pk)
        result["roofline_layernorm"] = extras.pop("roofline_layernorm")
        result["roofline_softmax"] = extras.pop("roofline_softmax")
        extras["c5"] = {"sequences_per_s": value, "us_per_layer": ms * 1e3 / c["layers"]}
        result["configs"] = extras
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from tests import oracle_lib
        result["cpu_baseline"] = cpu_baseline(oracle_lib.load(), c)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
