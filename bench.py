#!/usr/bin/env python
"""Benchmark of the encoder hot path on B200: one JSON line per run.

Workload (N=1): the tile-pruned BERT-base encoder layer of the `encoder_tile_test` configuration
(batch 16, seq 128, hidden 768, 12 heads, FFN 3072, fp16 storage, fp32 accumulate, seeded Bernoulli 16x16
tile mask). A step is one forward of the layer over the whole batch. `value` times the layer with inputs
resident in HBM; `e2e` times the public call with pinned host buffers (H2D of the batch, D2H of the result
inside the timed region). With N ranks each rank runs its own batch (weak scaling, no collective inside the
layer) and the output shards are gathered with one NCCL all-gather per step.

`--impl reference` runs the reference project's own CUDA kernels (library prebuilt from the reference
checkout under oracle/_ref/) on the same workload, composed in the reference's op order; if that library is
absent it times the fp32 CPU oracle instead.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_MODEL, NHEAD, D_FF, BATCH, SEQ = 768, 12, 3072, 16, 128
SWEEP = (0.5, 0.75, 0.9)
L2_FLUSH_BYTES = 256 << 20


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

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
        for s in self.samples:
            try:
                sm.append(float(s[0])); mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def make_layer_host(orc, sparsity, seed):
    from tests import util
    shapes = {"q": (D_MODEL, D_MODEL), "k": (D_MODEL, D_MODEL), "v": (D_MODEL, D_MODEL), "o": (D_MODEL, D_MODEL),
              "ffn1": (D_MODEL, D_FF), "ffn2": (D_FF, D_MODEL)}
    lin = {}
    for i, (name, (K, N)) in enumerate(shapes.items()):
        rp, ro, data, bias = util.make_tile_linear(orc, K, N, sparsity, seed + 10 * i, bernoulli=True)
        lin[name] = (rp, ro, data, bias, N, K)
    ln = ((np.ones(D_MODEL, np.float16), np.zeros(D_MODEL, np.float16)),
          (np.ones(D_MODEL, np.float16), np.zeros(D_MODEL, np.float16)))
    return lin, ln


def layer_flops(lin, tokens, batch, seq):
    gemm = sum(2.0 * tokens * 256 * len(v[1]) for v in lin.values())
    attn = 4.0 * seq * seq * D_MODEL * batch
    return gemm, attn


def cpu_baseline(orc, lin, ln, X):
    """The fp32 oracle (a CPU port of the layer) timed on the host cores over the full batch."""
    ol = {k: v[:5] for k, v in lin.items()}
    reps, t0 = 0, time.perf_counter()
    while True:
        orc.encoder_layer(X, ol, ln, [SEQ] * BATCH, D_MODEL, NHEAD)
        reps += 1
        el = time.perf_counter() - t0
        if el > 10.0 or reps >= 20:
            break
    return {"value": BATCH * reps / el, "unit": "sequences/s", "cores": orc.threads(), "kind": "port",
            "sample": f"{reps} full forwards of the {BATCH}x{SEQ} batch ({BATCH * SEQ} tokens), fp32 oracle with OpenMP"}


def run_reference(args, rank, world):
    """Reference arm: the reference's own CUDA kernels, or the CPU oracle when they are unavailable."""
    from tests import oracle_lib, util
    if rank != 0:
        return
    orc = oracle_lib.load()
    lin, ln = make_layer_host(orc, args.sparsity, seed=1234)
    X = util.activations(99, (BATCH * SEQ, D_MODEL))
    base = {"metric": "encoder sequences/sec (one tile-pruned BERT-base layer)", "unit": "sequences/s", "impl": "reference",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args)}
    ref = oracle_lib.load_ref()
    cpu = cpu_baseline(orc, lin, ln, X)
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if ref is None or not have_gpu:
        base.update({"value": cpu["value"], "ms_per_step": 1e3 * BATCH / cpu["value"], "cpu_baseline": cpu,
                     "reference_kind": "cpu-oracle-port",
                     "e2e": {"value": cpu["value"], "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        print(json.dumps(base))
        return
    import torch
    torch.cuda.set_device(0)
    T = BATCH * SEQ

    class Bsr(ctypes.Structure):
        _fields_ = [("row_ptr", ctypes.c_void_p), ("row_offset", ctypes.c_void_p), ("data", ctypes.c_void_p),
                    ("bias", ctypes.c_void_p)]
    keep = []
    arr = (Bsr * 6)()
    for i, name in enumerate(["q", "k", "v", "o", "ffn1", "ffn2"]):
        rp, ro, data, bias = lin[name][:4]
        ts = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (rp, ro, data, bias)]
        keep.append(ts)
        arr[i] = Bsr(*[t.data_ptr() for t in ts])
    lnd = [torch.from_numpy(a).cuda() for pair in ln for a in pair]
    mask = torch.zeros((SEQ, SEQ), dtype=torch.float16, device="cuda")
    x = torch.from_numpy(X).cuda()
    out = torch.zeros_like(x)
    buf = torch.zeros(8 * T * D_MODEL, dtype=torch.float16, device="cuda")
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    scale = ctypes.c_float(1.4426950408889634 / (D_MODEL // NHEAD) ** 0.5)   # base-2 kernel: true softmax
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def step():
        rc = ref.ref_encoder_tile_layer(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                        ctypes.c_void_p(buf.data_ptr()), arr, *[ctypes.c_void_p(t.data_ptr()) for t in lnd],
                                        ctypes.c_void_p(mask.data_ptr()), BATCH, SEQ, D_MODEL, NHEAD, D_FF, scale, st)
        assert rc == 0
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    times = []
    with ClockSampler(0) as cs:
        for _ in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); step(); e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    ms = sum(times) / len(times)
    # end to end with host buffers
    hx = torch.from_numpy(X).pin_memory()
    ho = torch.empty_like(hx).pin_memory()
    torch.cuda.synchronize()
    t_e2e = []
    for _ in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        x.copy_(hx, non_blocking=True); step(); ho.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        t_e2e.append(time.perf_counter() - t0)
    e2e = BATCH / (sum(t_e2e) / len(t_e2e))
    base.update({"value": BATCH / (ms * 1e-3), "ms_per_step": ms, "cpu_baseline": cpu,
                 "reference_kind": "reference CUDA kernels (oracle/_ref), linears+LayerNorm over all tokens, attention per sequence",
                 "clocks": cs.summary(),
                 "e2e": {"value": e2e, "unit": "sequences/s", "h2d_bytes_per_step": int(hx.numel() * 2),
                         "d2h_bytes_per_step": int(ho.numel() * 2)}})
    print(json.dumps(base))


def workload_config(args):
    return {"workload": f"config 2 (encoder_tile_test): one tile-pruned BERT-base encoder layer, batch {BATCH} x seq {SEQ}, "
                        f"hidden {D_MODEL}, {NHEAD} heads, FFN {D_FF}, Bernoulli 16x16 tile sparsity {args.sparsity} per GPU",
            "global_batch": BATCH * args.gpus, "seq_len": SEQ, "sparsity": args.sparsity,
            "parallelism": f"dp{args.gpus}" if args.gpus > 1 else "single",
            "l2": f"L2 flushed between timed steps by writing a {L2_FLUSH_BYTES >> 20} MiB buffer"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--sparsity", type=float, default=0.75)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sweep and the LayerNorm/softmax bandwidth legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import et_b200 as et
    from tests import oracle_lib, util
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    et.lib()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pk = peaks()
    orc = oracle_lib.load()
    T = BATCH * SEQ
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")

    def build(sparsity):
        lin, ln = make_layer_host(orc, sparsity, seed=1234)
        w = {n: et.TileWeight(v[5], v[4], T, v[2], v[0], v[1], v[3], is_gelu=(n == "ffn1")) for n, v in lin.items()}
        enc = et.Encoder(et.KIND_TILE, D_MODEL, SEQ, NHEAD, None, w["q"], w["k"], w["v"], w["o"], w["ffn1"], w["ffn2"],
                         (ln[0][0], ln[0][1], ln[1][0], ln[1][1]))
        return lin, ln, enc

    X = util.activations(99 + rank, (T, D_MODEL))
    x = torch.from_numpy(X).cuda()
    out = torch.zeros_like(x)
    scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, D_MODEL, T, BATCH, SEQ, NHEAD) // 2,
                          dtype=torch.float16, device="cuda")
    gathered = torch.zeros((world * T, D_MODEL), dtype=torch.float16, device="cuda") if world > 1 else None
    lens = [SEQ] * BATCH

    def timed_layer(enc, steps, warmup):
        def step():
            enc.run_batch(out, x, lens, scratch)
            if world > 1:
                dist.all_gather_into_tensor(gathered, out)
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        times = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); step(); e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        total = torch.tensor([sum(times)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.MAX)
        return total.item() / steps

    lin, ln, enc = build(args.sparsity)
    with ClockSampler(local_rank) as cs:
        ms = timed_layer(enc, args.steps, args.warmup)
    clocks = cs.summary()
    value = BATCH * world / (ms * 1e-3)
    gemm_flops, attn_flops = layer_flops(lin, T, BATCH, SEQ)

    # ---- end to end through the public call with host buffers (H2D + layer + D2H per step)
    hx = torch.from_numpy(X).pin_memory()
    ho = torch.empty_like(hx).pin_memory()
    t_e2e = []
    for i in range(args.warmup + args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        x.copy_(hx, non_blocking=True)
        enc.run_batch(out, x, lens, scratch)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)
        ho.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        if i >= args.warmup:
            t_e2e.append(time.perf_counter() - t0)
    e2e_t = torch.tensor([sum(t_e2e) / len(t_e2e)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e = {"value": BATCH * world / e2e_t.item(), "unit": "sequences/s", "h2d_bytes_per_step": int(hx.numel() * 2),
           "d2h_bytes_per_step": int(ho.numel() * 2)}

    # ---- roofline of the dominant kernel: the six tile-GEMM launches of the layer, timed alone
    w6 = {n: et.TileWeight(v[5], v[4], T, v[2], v[0], v[1], v[3]) for n, v in lin.items()}
    hbuf = torch.zeros((T, D_FF), dtype=torch.float16, device="cuda")
    ybuf = torch.zeros((T, D_FF), dtype=torch.float16, device="cuda")
    def gemms():
        for n in ("q", "k", "v", "o"):
            w6[n].run(ybuf.view(-1)[:T * D_MODEL].view(T, D_MODEL), x)
        w6["ffn1"].run(hbuf, x, gelu=True)
        w6["ffn2"].run(ybuf.view(-1)[:T * D_MODEL].view(T, D_MODEL), hbuf)
    for _ in range(3):
        gemms()
    torch.cuda.synchronize()
    gt = []
    for _ in range(max(10, args.steps // 2)):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); gemms(); e1.record()
        torch.cuda.synchronize()
        gt.append(e0.elapsed_time(e1))
    gemm_ms = sum(gt) / len(gt)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
    roofline = {"kernel": "tile_gemm_kernel (6 launches: Q,K,V,O,FFN1,FFN2)", "bound": "tensor", "achieved": achieved,
                "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"], "peak_source": pk["source"],
                "flops_per_launch_set": gemm_flops, "ms_per_launch_set": gemm_ms, "traffic": None,
                "dense_equivalent_tflops": achieved / max(1e-9, 1.0 - args.sparsity)}

    result = {"metric": "encoder sequences/sec (one tile-pruned BERT-base layer)", "value": value, "unit": "sequences/s",
              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "us_per_layer": ms * 1e3,
              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
              "config": workload_config(args), "clocks": clocks, "e2e": e2e, "gpu_launches": 9 * args.steps,
              "roofline": roofline,
              "layer_tflops": (gemm_flops + attn_flops) / (ms * 1e-3) / 1e12}

    if rank == 0 and not args.no_extras:
        extras = {}
        # sparsity sweep of the same layer
        for s in SWEEP:
            if abs(s - args.sparsity) < 1e-9:
                extras[str(s)] = {"us_per_layer": ms * 1e3, "sequences_per_s": BATCH / (ms * 1e-3)}
                continue
            _, _, e2 = build(s)
            m2 = timed_layer(e2, max(10, args.steps // 2), 3) if world == 1 else None
            if m2:
                extras[str(s)] = {"us_per_layer": m2 * 1e3, "sequences_per_s": BATCH / (m2 * 1e-3)}
        result["sweep"] = extras
        # bandwidth kernels on inputs larger than L2
        rows, dm = 131072, 1024
        a = torch.randn((rows, dm), device="cuda").half(); b = torch.randn((rows, dm), device="cuda").half()
        g = torch.ones(dm, dtype=torch.float16, device="cuda"); be = torch.zeros(dm, dtype=torch.float16, device="cuda")
        for _ in range(3):
            et.skip_layernorm(a, b, g, be)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            et.skip_layernorm(a, b, g, be)
        e1.record(); torch.cuda.synchronize()
        ln_ms = e0.elapsed_time(e1) / 10
        gbs = 6.0 * dm * rows / (ln_ms * 1e-3) / 1e9
        result["roofline_layernorm"] = {"kernel": "skip_layernorm_vec<4>", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"],
                                        "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "rows": rows, "size": dm}
        del a, b
        nmat, L = 16 * 64, 512
        S = torch.randn((nmat, L, L), device="cuda").half()
        for _ in range(3):
            et.softmax_mask(S)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            et.softmax_mask(S)
        e1.record(); torch.cuda.synchronize()
        sm_ms = e0.elapsed_time(e1) / 10
        gbs = 4.0 * L * L * nmat / (sm_ms * 1e-3) / 1e9
        result["roofline_softmax"] = {"kernel": "softmax_mask_vec<2>", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"],
                                      "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "matrices": nmat, "seq_len": L}
        del S
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(orc, lin, ln, X)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
