#!/usr/bin/env python
"""Benchmark of the encoder hot path on B200: one JSON line per run.

Workload (N=1): the tile-pruned BERT-base encoder layer of the `encoder_tile_test` configuration
(batch 16, seq 128, hidden 768, 12 heads, FFN 3072, fp16 storage, fp32 accumulate, seeded Bernoulli 16x16
tile mask). A step is one forward of the layer over the whole batch. `value` times the layer with inputs
resident in HBM; `e2e` times the public call with pinned host buffers (H2D of every step's batch and D2H of its
result inside the timed region, as a three-stage pipeline on separate streams; the figure with a host
synchronisation after every step is reported beside it). `--streams` independent batches (default 6) are in
flight per GPU, one CUDA stream each: the layer's launches are short and rarely fill the GPU, so concurrent
batches use the SMs a single batch leaves idle, and the weights are packed for the least SM time per launch
(`et_set_tuning_goal`); `us_per_layer` is the latency with one batch at a time on weights packed for the shortest
single launch. The reference arm runs with the same number of streams. With N ranks each rank runs its own batch (weak scaling, no collective inside the
layer) and the output shards are gathered with one NCCL all-gather per step.

Cold-cache rule: the step visits INSTANCES independent copies of the workload (own weights, activations,
scratch; about 25 MB each, 300 MB in total) round-robin, so no step finds its inputs in the 126 MB L2.

`--impl reference` runs the reference project's own CUDA kernels (library prebuilt from the reference
checkout under oracle/_ref/) on the same workload, composed in the reference's op order; if that library is
absent it times the fp32 CPU oracle instead.
"""
import argparse
import collections
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
T = BATCH * SEQ
SWEEP = (0.5, 0.75, 0.9)
INSTANCES = 12
METRIC = "encoder sequences/sec (one tile-pruned BERT-base layer)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the GPU is under load."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
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
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def set_shape(args):
    """Other shapes of the same tile-pruned layer (e.g. --batch 1 --sparsity 0 for the dense single-sequence case,
    --batch 32 --seq 512 --d-model 1024 --heads 16 --ff 4096 --sparsity 0.8 for a BERT-large shard). The instance
    count shrinks with the size of an instance but the instances together always exceed L2."""
    global D_MODEL, NHEAD, D_FF, BATCH, SEQ, T, INSTANCES
    D_MODEL, NHEAD, D_FF, BATCH, SEQ = args.d_model, args.heads, args.ff, args.batch, args.seq
    T = BATCH * SEQ
    per_instance = 7 * T * D_MODEL * 2 + (4 * D_MODEL * D_MODEL + 2 * D_MODEL * D_FF) * 2 * (1.0 - args.sparsity)
    INSTANCES = int(max(2, min(12, -(-300e6 // per_instance))))


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


def layer_flops(lin):
    gemm = sum(2.0 * T * 256 * len(v[1]) for v in lin.values())
    attn = 4.0 * SEQ * SEQ * D_MODEL * BATCH
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
            "sample": f"{reps} full forwards of the {BATCH}x{SEQ} batch ({T} tokens), fp32 oracle with OpenMP"}


def workload_config(args):
    name = "config 2 (encoder_tile_test)" if (D_MODEL, NHEAD, D_FF, BATCH, SEQ) == (768, 12, 3072, 16, 128) else "encoder_tile_test shape"
    return {"workload": f"{name}: one tile-pruned BERT encoder layer, batch {BATCH} x seq {SEQ}, "
                        f"hidden {D_MODEL}, {NHEAD} heads, FFN {D_FF}, Bernoulli 16x16 tile sparsity {args.sparsity} per GPU",
            "global_batch": BATCH * args.gpus, "seq_len": SEQ, "sparsity": args.sparsity,
            "parallelism": f"dp{args.gpus}" if args.gpus > 1 else "single",
            "batches_in_flight": f"{args.streams} independent batches per GPU on {args.streams} CUDA streams (step i on stream i mod "
                                 f"{args.streams}); us_per_layer is the latency with one batch at a time",
            "gather": (f"NCCL all-gather of the output shards, the outputs of {args.gather_every} consecutive steps per collective, "
                       "asynchronous, joined inside the timed region") if args.gpus > 1 else "none",
            "l2": f"inputs larger than L2: {INSTANCES} independent instances of the layer (weights, activations, scratch, about "
                  f"{7 * T * D_MODEL * 2 / 1e6:.0f} MB each) visited round-robin"}


def timed(step, steps, finish=None, start=None):
    """`steps` calls of step(i) between two CUDA events on the current stream; returns ms per step.
    `start` (optional) runs right after the opening event (side streams wait for it there), `finish` (optional)
    runs before the closing event, e.g. to join side streams and collectives still in flight."""
    import torch
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if start:
        start()
    for i in range(steps):
        step(i)
    if finish:
        finish()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def pipelined_e2e(torch, n_steps, n_inst, h2d, compute, d2h, depth, comp_streams):
    """Seconds per step of a three-stage pipeline over `n_inst` independent buffer sets: the host-to-device copy of
    step i+1 and the device-to-host copy of step i-1 run on their own streams under the layers of the steps in
    between (set k always computes on comp_streams[k mod len]). Every step's input is copied from pinned host
    memory and its result is copied back inside the timed region; the host waits for the result of step i-depth
    before it enqueues step i (a server consuming results, and a bound on the work in flight).

    h2d[k] / d2h[k] = (dst pointer, src pointer, bytes); compute(k) launches set k's layer on its stream. Copies
    and events go through the CUDA runtime directly (ctypes): the host's enqueue cost per step would otherwise
    exceed the device time of a step."""
    rt = ctypes.CDLL("libcudart.so.12")
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    rt.cudaMemcpyAsync.argtypes = [vp, vp, sz, ctypes.c_int, vp]
    rt.cudaEventRecord.argtypes = [vp, vp]
    rt.cudaStreamWaitEvent.argtypes = [vp, vp, ctypes.c_uint]
    rt.cudaEventSynchronize.argtypes = [vp]
    rt.cudaEventCreateWithFlags.argtypes = [ctypes.POINTER(vp), ctypes.c_uint]
    rt.cudaEventDestroy.argtypes = [vp]

    def chk(rc):
        if rc != 0:
            raise RuntimeError(f"CUDA runtime call failed with error {rc}")

    def new_event():
        ev = vp()
        chk(rt.cudaEventCreateWithFlags(ctypes.byref(ev), 2))   # cudaEventDisableTiming
        return ev
    t_in, t_out = torch.cuda.Stream(), torch.cuda.Stream()
    s_in, s_out = vp(t_in.cuda_stream), vp(t_out.cuda_stream)
    comps = [vp(st.cuda_stream) for st in comp_streams]
    ev_in = [new_event() for _ in range(n_inst)]
    ev_comp = [new_event() for _ in range(n_inst)]
    ev_out = [new_event() for _ in range(n_inst)]
    used = [False] * n_inst

    def step(i):
        k = i % n_inst
        if i >= depth and used[(i - depth) % n_inst]:
            chk(rt.cudaEventSynchronize(ev_out[(i - depth) % n_inst]))
        if used[k]:
            chk(rt.cudaStreamWaitEvent(s_in, ev_comp[k], 0))    # the previous layer on this set has read its input
        chk(rt.cudaMemcpyAsync(h2d[k][0], h2d[k][1], h2d[k][2], 1, s_in))
        chk(rt.cudaEventRecord(ev_in[k], s_in))
        s_comp = comps[k % len(comps)]
        chk(rt.cudaStreamWaitEvent(s_comp, ev_in[k], 0))
        if used[k]:
            chk(rt.cudaStreamWaitEvent(s_comp, ev_out[k], 0))   # the previous result has left the output buffer
        compute(k)
        chk(rt.cudaEventRecord(ev_comp[k], s_comp))
        chk(rt.cudaStreamWaitEvent(s_out, ev_comp[k], 0))
        chk(rt.cudaMemcpyAsync(d2h[k][0], d2h[k][1], d2h[k][2], 2, s_out))
        chk(rt.cudaEventRecord(ev_out[k], s_out))
        used[k] = True

    torch.cuda.synchronize()
    for i in range(2 * n_inst):
        step(i)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n_steps):
        step(i)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / n_steps
    for ev in ev_in + ev_comp + ev_out:
        rt.cudaEventDestroy(ev)
    return dt


def run_reference(args, rank):
    """Reference arm: the reference's own CUDA kernels, or the CPU oracle when they are unavailable."""
    from tests import oracle_lib, util
    if rank != 0:
        return
    orc = oracle_lib.load()
    lin, ln = make_layer_host(orc, args.sparsity, seed=1234)
    X = util.activations(99, (T, D_MODEL))
    base = {"metric": METRIC, "unit": "sequences/s", "impl": "reference", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": workload_config(args)}
    ref = oracle_lib.load_ref()
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    cpu = cpu_baseline(orc, lin, ln, X) if (ref is None or not have_gpu or not args.no_cpu_baseline) else None
    if ref is None or not have_gpu:
        base.update({"value": cpu["value"], "ms_per_step": 1e3 * BATCH / cpu["value"], "cpu_baseline": cpu,
                     "reference_kind": "fp32 CPU oracle (the reference ships no CPU path and its CUDA library is not built here)",
                     "e2e": {"value": cpu["value"], "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        print(json.dumps(base))
        return
    import torch
    torch.cuda.set_device(0)

    class Bsr(ctypes.Structure):
        _fields_ = [("row_ptr", ctypes.c_void_p), ("row_offset", ctypes.c_void_p), ("data", ctypes.c_void_p),
                    ("bias", ctypes.c_void_p)]

    class RefInstance:
        def __init__(self, idx):
            self.keep, self.arr = [], (Bsr * 6)()
            for i, name in enumerate(["q", "k", "v", "o", "ffn1", "ffn2"]):
                ts = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in lin[name][:4]]
                self.keep.append(ts)
                self.arr[i] = Bsr(*[t.data_ptr() for t in ts])
            self.lnd = [torch.from_numpy(a).cuda() for pair in ln for a in pair]
            self.mask = torch.zeros((SEQ, SEQ), dtype=torch.float16, device="cuda")
            self.X = util.activations(99 + 1000 * idx, (T, D_MODEL))
            self.x = torch.from_numpy(self.X).cuda()
            self.out = torch.zeros_like(self.x)
            self.buf = torch.zeros(8 * T * D_MODEL, dtype=torch.float16, device="cuda")

    insts = [RefInstance(i) for i in range(INSTANCES)]
    scale = ctypes.c_float(1.4426950408889634 / (D_MODEL // NHEAD) ** 0.5)   # base-2 kernel: true softmax
    vp = ctypes.c_void_p
    # the same number of independent batches in flight as the native arm, one stream each
    NS = max(d for d in range(1, max(1, args.streams) + 1) if INSTANCES % d == 0)
    main_stream = torch.cuda.current_stream()
    streams = [main_stream] + [torch.cuda.Stream() for _ in range(NS - 1)]

    def run_on(i, stream):
        it = insts[i % INSTANCES]
        rc = ref.ref_encoder_tile_layer(vp(it.out.data_ptr()), vp(it.x.data_ptr()), vp(it.buf.data_ptr()), it.arr,
                                        *[vp(t.data_ptr()) for t in it.lnd], vp(it.mask.data_ptr()), BATCH, SEQ,
                                        D_MODEL, NHEAD, D_FF, scale, vp(stream.cuda_stream))
        assert rc == 0

    def step(i):   # on whatever stream is current (end-to-end loops)
        run_on(i, torch.cuda.current_stream())

    def fork():
        for s_ in streams[1:]:
            s_.wait_stream(main_stream)

    def join():
        for s_ in streams[1:]:
            main_stream.wait_stream(s_)

    def mstep(i):
        run_on(i, streams[i % NS])
    with ClockSampler(0) as cs:
        timed(mstep, max(args.warmup, 300), join, fork)
        ms = timed(mstep, args.steps, join, fork)
        ms_one = timed(step, max(100, args.steps // 4)) if NS > 1 else ms
    hx = [torch.from_numpy(it.X).pin_memory() for it in insts]
    ho = [torch.empty_like(h).pin_memory() for h in hx]
    n_e2e = min(args.steps, 300)

    def e2e_step(i):
        it = insts[i % INSTANCES]
        it.x.copy_(hx[i % INSTANCES], non_blocking=True)
        step(i)
        ho[i % INSTANCES].copy_(it.out, non_blocking=True)
        torch.cuda.synchronize()
    for i in range(INSTANCES):
        e2e_step(i)
    t0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    e2e_sync = BATCH / ((time.perf_counter() - t0) / n_e2e)
    nbytes = hx[0].numel() * 2
    e2e = BATCH / pipelined_e2e(torch, n_e2e, INSTANCES,
                                [(vp(insts[k].x.data_ptr()), vp(hx[k].data_ptr()), nbytes) for k in range(INSTANCES)],
                                lambda k: run_on(k, streams[k % NS]),
                                [(vp(ho[k].data_ptr()), vp(insts[k].out.data_ptr()), nbytes) for k in range(INSTANCES)],
                                depth=2 * NS, comp_streams=streams)
    base.update({"value": BATCH / (ms * 1e-3), "ms_per_step": ms, "us_per_layer": ms_one * 1e3,
                 "us_per_step_throughput": ms * 1e3, "batches_in_flight": NS, "cpu_baseline": cpu,
                 "reference_kind": "the reference's CUDA kernels (oracle/_ref): linears and LayerNorms once over all tokens, "
                                   "attention once per sequence, one stream, no host synchronisation",
                 "clocks": cs.summary(),
                 "e2e": {"value": e2e, "unit": "sequences/s", "h2d_bytes_per_step": int(hx[0].numel() * 2),
                         "d2h_bytes_per_step": int(ho[0].numel() * 2), "steps": n_e2e,
                         "how": "three-stage pipeline (H2D, layer, D2H on separate streams), every step's input and "
                                "result cross PCIe inside the timed region",
                         "synchronous_per_step": e2e_sync}})
    print(json.dumps(base))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5000)
    ap.add_argument("--warmup", type=int, default=3000)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--sparsity", type=float, default=0.75)
    ap.add_argument("--batch", type=int, default=BATCH, help="sequences per GPU (other configurations of the tile layer)")
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--d-model", type=int, default=D_MODEL)
    ap.add_argument("--heads", type=int, default=NHEAD)
    ap.add_argument("--ff", type=int, default=D_FF)
    ap.add_argument("--streams", type=int, default=6,
                    help="independent batches in flight per GPU, one CUDA stream each (1 = one batch at a time)")
    ap.add_argument("--gather-every", type=int, default=12,
                    help="multi-GPU: output shards of this many steps travel in one all-gather (must divide the instance count)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sweep and the LayerNorm/softmax bandwidth legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    set_shape(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
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
    lens = [SEQ] * BATCH
    # Independent batches run concurrently, one CUDA stream each (step i on stream i mod NS): the layer's launches
    # are short and seldom fill 148 SMs, so a second and third batch use what the first leaves idle.
    NS = max(d for d in range(1, max(1, args.streams) + 1) if INSTANCES % d == 0)   # an instance stays on one stream
    # None of them is the legacy default stream: the layer's CUDA-graph replay needs a capturable stream.
    main_stream = torch.cuda.current_stream()
    streams = [torch.cuda.Stream() for _ in range(NS)]
    # Output shards are gathered over NVLink with NCCL all-gathers on a stream of their own: the next steps' layers
    # do not wait for them. The outputs of GE consecutive steps land side by side in one of three staging buffers
    # and travel in one collective (every output row is gathered inside the timed region; fewer, larger
    # collectives take fewer SMs away from the layer's kernels). A staging buffer is written again only after the
    # collective that read it has completed (events); everything is joined before the closing event of a timed
    # region.
    GE = args.gather_every if world > 1 else 1
    if world > 1 and (GE < 1 or INSTANCES % GE):
        GE = 1
    stage = [torch.zeros((GE * T, D_MODEL), dtype=torch.float16, device="cuda") for _ in range(3)] if world > 1 else None
    gathered = [torch.zeros((world * GE * T, D_MODEL), dtype=torch.float16, device="cuda") for _ in range(4)] if world > 1 else None
    gstream = torch.cuda.Stream() if world > 1 else None
    ev_step = [torch.cuda.Event() for _ in range(3 * GE)]   # step finished writing its slice of a staging buffer
    ev_free = [torch.cuda.Event() for _ in range(3)]        # the collective that read a staging buffer has completed
    gathers_issued = [0]
    open_group = [None]   # a group whose last step has not run yet

    def gather(group, slots):
        with torch.cuda.stream(gstream):
            for sl in range(slots):
                gstream.wait_event(ev_step[(group % 3) * GE + sl])
            work = dist.all_gather_into_tensor(gathered[group % 4], stage[group % 3], async_op=True)
            work.wait()                       # the gather stream waits for the collective, not the host
            ev_free[group % 3].record(gstream)
        gathers_issued[0] += 1

    def fork():
        for st in streams:
            st.wait_stream(main_stream)
        if gstream is not None:
            gstream.wait_stream(main_stream)

    def join():
        if open_group[0] is not None:   # the step count was not a multiple of GE: gather the partial group too
            g, slots = open_group[0]
            gather(g, slots)
            open_group[0] = None
        for st in streams:
            main_stream.wait_stream(st)
        if gstream is not None:
            main_stream.wait_stream(gstream)

    class Instance:
        """One independent copy of the workload: its own weights, input, output and scratch."""
        def __init__(self, sparsity, idx):
            self.lin, self.ln = make_layer_host(orc, sparsity, seed=1234)
            w = {n: et.TileWeight(v[5], v[4], T, v[2], v[0], v[1], v[3], is_gelu=(n == "ffn1"))
                 for n, v in self.lin.items()}
            self.enc = et.Encoder(et.KIND_TILE, D_MODEL, SEQ, NHEAD, None, w["q"], w["k"], w["v"], w["o"], w["ffn1"],
                                  w["ffn2"], (self.ln[0][0], self.ln[0][1], self.ln[1][0], self.ln[1][1]))
            self.X = util.activations(99 + rank + 1000 * idx, (T, D_MODEL))
            self.x = torch.from_numpy(self.X).cuda()
            self.out = torch.zeros_like(self.x)
            self.scratch = torch.zeros(et.encoder_batch_buffer_size(et.KIND_TILE, D_MODEL, T, BATCH, SEQ, NHEAD) // 2,
                                       dtype=torch.float16, device="cuda")

    lens_np = np.ascontiguousarray(lens, dtype=np.int32)
    run_batch_c = et.lib().et_encoder_run_batch
    vp = ctypes.c_void_p

    def layer_step(insts, ns):
        # The public C entry point, called with arguments converted once: instance k always runs on stream k mod ns
        # and (multi-GPU) always writes slice k mod GE of a staging buffer, so there is one constant call per
        # (staging buffer, instance); the layer keeps one replayable graph per output address.
        calls = []
        for b in range(3 if world > 1 else 1):
            row = []
            for k, it in enumerate(insts):
                out = it.out if world == 1 else stage[b][(k % GE) * T:((k % GE) + 1) * T]
                row.append((it.enc._h, vp(out.data_ptr()), vp(it.x.data_ptr()), vp(lens_np.ctypes.data), vp(0), ctypes.c_int(BATCH),
                            vp(it.scratch.data_ptr()), ctypes.c_size_t(it.scratch.numel() * 2),
                            vp(streams[k % ns].cuda_stream)))
            calls.append(row)

        def step(i):
            k = i % len(insts)
            st = streams[k % ns]
            if world > 1:
                group, slot = divmod(i, GE)
                if group >= 3:
                    st.wait_event(ev_free[group % 3])   # the collective of group - 3 has read this buffer
            rc = run_batch_c(*calls[group % 3 if world > 1 else 0][k])
            if rc:
                raise et.EtError(rc, et.lib().et_last_error().decode())
            if world > 1:
                ev_step[(group % 3) * GE + slot].record(st)
            if world > 1:
                open_group[0] = (group, slot + 1)
                if slot == GE - 1:
                    gather(group, GE)
                    open_group[0] = None
        return step

    def measure(insts, steps, warmup, ns=None):
        step = layer_step(insts, NS if ns is None else ns)
        # direct run, graph capture and first replay of every instance (on every staging buffer it writes to)
        timed(step, 3 * len(insts) * (3 if world > 1 else 1), join, fork)
        timed(step, warmup, join, fork)
        if world > 1:
            dist.barrier()
        ms = timed(step, steps, join, fork)
        if world > 1:
            dist.barrier()
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    # With several batches in flight the SMs are busy anyway, so the weights are packed for the least SM time per
    # launch (fewer, larger tiles); the latency of one batch at a time is measured on weights packed for the
    # shortest single launch (the library's default).
    et.set_tuning_goal("throughput" if NS > 1 else "latency")
    insts = [Instance(args.sparsity, i) for i in range(INSTANCES)]
    lin, ln, X = insts[0].lin, insts[0].ln, insts[0].X
    with ClockSampler(local_rank) as cs:
        ms = measure(insts, args.steps, args.warmup)
    clocks = cs.summary()
    ms_one = ms
    if NS > 1:
        et.set_tuning_goal("latency")
        lat = [Instance(args.sparsity, i) for i in range(INSTANCES)]
        ms_one = measure(lat, max(300, args.steps // 4), 100, ns=1)
        del lat
        et.set_tuning_goal("throughput")
    value = BATCH * world / (ms * 1e-3)
    gemm_flops, attn_flops = layer_flops(lin)

    # ---- end to end through the public call with host buffers (H2D + layer + D2H per step)
    hx = [torch.from_numpy(it.X).pin_memory() for it in insts]
    ho = [torch.empty_like(h).pin_memory() for h in hx]
    n_e2e = min(args.steps, 500)

    def e2e_step(i):
        it = insts[i % INSTANCES]
        with torch.cuda.stream(streams[0]):
            it.x.copy_(hx[i % INSTANCES], non_blocking=True)
            it.enc.run_batch(it.out, it.x, lens, it.scratch)
            if world > 1:
                dist.all_gather_into_tensor(gathered[0][:world * T], it.out)
            ho[i % INSTANCES].copy_(it.out, non_blocking=True)
        torch.cuda.synchronize()          # the caller needs the result on the host before its next batch
    for i in range(INSTANCES):
        e2e_step(i)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    e2e_sync_s = (time.perf_counter() - t0) / n_e2e

    e2e_calls = [(it.enc._h, vp(it.out.data_ptr()), vp(it.x.data_ptr()), vp(lens_np.ctypes.data), vp(0), ctypes.c_int(BATCH),
                  vp(it.scratch.data_ptr()), ctypes.c_size_t(it.scratch.numel() * 2), vp(streams[k % NS].cuda_stream))
                 for k, it in enumerate(insts)]

    def e2e_compute(k):
        rc = run_batch_c(*e2e_calls[k])
        if rc:
            raise et.EtError(rc, et.lib().et_last_error().decode())
        if world > 1:
            with torch.cuda.stream(streams[k % NS]):
                dist.all_gather_into_tensor(gathered[0][:world * T], insts[k].out)
    if world > 1:
        dist.barrier()
    nbytes = hx[0].numel() * 2
    e2e_s = pipelined_e2e(torch, n_e2e, INSTANCES,
                          [(vp(insts[k].x.data_ptr()), vp(hx[k].data_ptr()), nbytes) for k in range(INSTANCES)], e2e_compute,
                          [(vp(ho[k].data_ptr()), vp(insts[k].out.data_ptr()), nbytes) for k in range(INSTANCES)],
                          depth=2 * NS, comp_streams=streams)
    if world > 1:
        t = torch.tensor([e2e_s, e2e_sync_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, e2e_sync_s = t[0].item(), t[1].item()
    e2e = {"value": BATCH * world / e2e_s, "unit": "sequences/s", "h2d_bytes_per_step": int(hx[0].numel() * 2),
           "d2h_bytes_per_step": int(ho[0].numel() * 2), "steps": n_e2e,
           "how": "three-stage pipeline (H2D, layer, D2H on separate streams) through et_encoder_run_batch, every "
                  "step's input and result cross PCIe inside the timed region",
           "synchronous_per_step": BATCH * world / e2e_sync_s}

    # ---- roofline of the dominant kernel: the tile-GEMM launches of the layer (fused Q|K|V, output, FFN1, FFN2),
    # timed alone through the C ABI, rotating over independent weight/activation sets (larger than L2 in total),
    # with the same number of sets in flight on the same streams as in the timed region of `value`
    raw = et.lib()
    sets = []
    for it in insts:
        w = {n: et.TileWeight(v[5], v[4], T, v[2], v[0], v[1], v[3]) for n, v in it.lin.items()}
        qkv_rp = np.concatenate([it.lin["q"][0], it.lin["k"][0][1:] + it.lin["q"][0][-1],
                                 it.lin["v"][0][1:] + it.lin["q"][0][-1] + it.lin["k"][0][-1]]).astype(np.int32)
        qkv = et.TileWeight(D_MODEL, 3 * D_MODEL, T, np.concatenate([it.lin[n][2] for n in "qkv"]), qkv_rp,
                            np.concatenate([it.lin[n][1] for n in "qkv"]), np.concatenate([it.lin[n][3] for n in "qkv"]))
        sets.append((qkv, w["o"], w["ffn1"], w["ffn2"], it.x,
                     torch.zeros((T, D_FF), dtype=torch.float16, device="cuda"),
                     torch.zeros((T, D_FF), dtype=torch.float16, device="cuda")))

    gemm_calls = []
    for k, (qkv, o, f1, f2, xx, hbuf, ybuf) in enumerate(sets):
        st = vp(streams[k % NS].cuda_stream)
        ti = ctypes.c_int(T)
        gemm_calls.append(((qkv._h, vp(ybuf.data_ptr()), vp(xx.data_ptr()), ti, ctypes.c_int(0), st),
                           (o._h, vp(hbuf.data_ptr()), vp(xx.data_ptr()), ti, ctypes.c_int(0), st),
                           (f1._h, vp(hbuf.data_ptr()), vp(xx.data_ptr()), ti, ctypes.c_int(1), st),
                           (f2._h, vp(ybuf.data_ptr()), vp(hbuf.data_ptr()), ti, ctypes.c_int(0), st)))

    def gemms(i):
        for c in gemm_calls[i % len(gemm_calls)]:
            raw.et_tile_linear(*c)
    timed(gemms, 2 * len(sets), join, fork)
    gemm_ms = timed(gemms, max(100, args.steps // 10), join, fork)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
    roofline = {"kernel": "tile_gemm_kernel (4 launches per layer: fused Q|K|V, output, FFN1+GELU, FFN2)", "bound": "tensor",
                "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                "peak_source": pk["source"] + " (bf16 burst)", "flops_per_launch_set": gemm_flops,
                "ms_per_launch_set": gemm_ms, "traffic": None,
                "dense_equivalent_tflops": achieved / max(1e-9, 1.0 - args.sparsity),
                "sets_in_flight": NS,
                "note": "algorithmic FLOPs count kept tiles only (2*T*256*ntile); ms_per_launch_set is wall time per set "
                        "of four launches with sets_in_flight independent sets in flight on separate streams; at 2048 "
                        "tokens a launch is bound by per-CTA latency (prologue, slot-ring hops, epilogue), see DESIGN.md"}

    result = {"metric": METRIC, "value": value, "unit": "sequences/s", "n_gpus": world, "steps": args.steps,
              "warmup": args.warmup, "ms_per_step": ms, "us_per_layer": ms_one * 1e3,
              "us_per_step_throughput": ms * 1e3, "batches_in_flight": NS, "higher_is_better": True,
              "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
              "config": workload_config(args), "clocks": clocks, "e2e": e2e, "gpu_launches": 7 * args.steps,
              "launches_per_step": "7: fused Q|K|V tile GEMM, attention, output tile GEMM, LayerNorm, FFN1 tile GEMM (GELU), "
                                   "FFN2 tile GEMM, LayerNorm; replayed as one CUDA graph",
              "roofline": roofline, "layer_tflops": (gemm_flops + attn_flops) / (ms * 1e-3) / 1e12}

    if rank == 0 and not args.no_extras and world == 1:
        sweep = {}
        for s in SWEEP:
            if abs(s - args.sparsity) < 1e-9:
                sweep[str(s)] = {"us_per_step": ms * 1e3, "sequences_per_s": BATCH / (ms * 1e-3)}
                continue
            i2 = [Instance(s, i) for i in range(INSTANCES)]
            m2 = measure(i2, max(300, args.steps // 4), 100)
            sweep[str(s)] = {"us_per_step": m2 * 1e3, "sequences_per_s": BATCH / (m2 * 1e-3)}
            del i2
        result["sweep"] = sweep
        # bandwidth kernels on inputs larger than L2
        rows, dm = 131072, 1024
        a = torch.randn((rows, dm), device="cuda").half(); b = torch.randn((rows, dm), device="cuda").half()
        g = torch.ones(dm, dtype=torch.float16, device="cuda"); be = torch.zeros(dm, dtype=torch.float16, device="cuda")
        timed(lambda i: et.skip_layernorm(a, b, g, be), 3)
        ln_ms = timed(lambda i: et.skip_layernorm(a, b, g, be), 20)
        gbs = 6.0 * dm * rows / (ln_ms * 1e-3) / 1e9
        result["roofline_layernorm"] = {"kernel": "skip_layernorm_vec<4>", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"],
                                        "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "rows": rows, "size": dm,
                                        "bytes_per_row": 6 * dm}
        del a, b
        nmat, L = 16 * 64, 512
        S = torch.randn((nmat, L, L), device="cuda").half()
        timed(lambda i: et.softmax_mask(S), 3)
        sm_ms = timed(lambda i: et.softmax_mask(S), 20)
        gbs = 4.0 * L * L * nmat / (sm_ms * 1e-3) / 1e9
        result["roofline_softmax"] = {"kernel": "softmax_mask_vec<2>", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"],
                                      "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "matrices": nmat, "seq_len": L,
                                      "bytes_per_matrix": 4 * L * L}
        del S
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(orc, lin, ln, X)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
