#!/usr/bin/env python
"""Benchmark of the quantized-linear path: one step = one decode pass (M activation rows)
through every quantized linear of the named model's stack, weights resident in HBM.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--rows 1]
  python bench.py --impl reference ...      # the CPU scheme on the host cores
  python bench.py --workload cfg2 --rows 2048 --mode TENSOR_CORE --xdtype bf16 --no-head   # prefill (config.tflops)
  torchrun ... bench.py --gpus N --workload cfg5 --tp --rows 64 --mode AUTO               # tensor-parallel pass

Prints ONE JSON line. `value` is weight bytes streamed per second over all GPUs (the
"QMatMul weight GB/s" metric); `e2e` is the same pass driven through the host-buffer entry
(activations copied in, results copied out, every linear); `roofline` describes the dominant
GEMV kernel; `cpu_baseline` is the CPU restatement of the reference scheme on this host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tur_b200.workloads import SEED, TYPE_NAMES, WORKLOADS, Weight  # noqa: E402

METRIC = "qmatmul_decode_weight_bandwidth"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, keyed by
# (members of the launch, workload, rows); absent = never captured = reported as null
NCU_TRAFFIC_BYTES = {(("ffn_gate", "ffn_up"), "cfg2", 1): 56736512}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_tensor_peak():
    """Burst bf16/f16 dense TFLOP/s (the denominator for a kernel timed alone)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


# ------------------------------------------------------------------ synthetic inputs

def gen_weight_blocks(w: Weight, seed: int, max_rows: int = 16384) -> np.ndarray:
    """Seeded N(0, 0.02) f32 weights quantized by the CPU quantizer; beyond max_rows the
    distinct rows repeat (the bytes streamed are what matters for timing)."""
    import oracle
    rng = np.random.default_rng(seed)
    rows = min(w.n, max_rows)
    f = (rng.standard_normal((rows, w.k), dtype=np.float32) * np.float32(0.02))
    blocks = oracle.quantize(w.dtype, f)
    if rows < w.n:
        reps = -(-w.n // rows)
        blocks = np.tile(blocks, (reps, 1))[: w.n]
    return np.ascontiguousarray(blocks)


def gen_activations(m: int, k: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)


# ------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        if self._thread:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------ CPU arm

def cpu_sample_weights(wl):
    """The bounded sample both CPU legs time: 1/layers of a pass, i.e. one layer's seven linears
    plus the same share of the head's rows, so that the weight mix of the pass is kept."""
    ws = [(w, gen_weight_blocks(w, SEED + i)) for i, w in enumerate(wl.per_layer)]
    if wl.head is not None:
        rows = max(16, (wl.head.n // wl.layers) // 16 * 16)
        hw = Weight(wl.head.name, rows, wl.head.k, wl.head.dtype, wl.head.source, wl.head.parallel)
        ws.append((hw, gen_weight_blocks(hw, SEED + 999)))
    return ws


def cpu_scheme_timing(wl, m: int, steps: int, warmup: int = 2, step_seconds: float = 0.5):
    """Times the CPU restatement of the reference's QMatMul::forward scheme (oracle/) with all
    host threads. One step = the bounded sample repeated `reps` times, reps chosen during the
    warm-up so that a step takes about `step_seconds`; exactly `steps` steps are timed as one
    region. Returns (GB/s of weight bytes, cores, sample text, ms per step, bytes per step)."""
    import oracle
    ws = cpu_sample_weights(wl)
    xs = {src: gen_activations(m, k, SEED + 10**6 + m + j) for j, (src, k) in
          enumerate(sorted({(w.source, w.k) for w, _ in ws}))}
    sample_bytes = sum(w.nbytes for w, _ in ws)

    # all host threads this process may use, also under torchrun (which sets OMP_NUM_THREADS=1)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)

    def one_pass():
        for w, b in ws:
            oracle.qmatmul(w.dtype, b, w.n, w.k, xs[w.source], nthreads=cores)

    one_pass()
    t0 = time.perf_counter()
    one_pass()
    reps = int(min(100, max(1, round(step_seconds / max(time.perf_counter() - t0, 1e-6)))))
    for _ in range(max(1, warmup)):
        for _ in range(reps):
            one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        for _ in range(reps):
            one_pass()
    per_step = (time.perf_counter() - t0) / steps
    sample = (f"{reps} x 1/{wl.layers} of a {wl.name} pass per step: one layer's 7 linears"
              + (f" + {ws[-1][0].n} of the lm_head's {wl.head.n} rows" if wl.head is not None else "")
              + f" ({sample_bytes / 1e6:.1f} MB of blocks each), M={m}, {steps} steps timed as one region")
    return reps * sample_bytes / per_step / 1e9, cores, sample, per_step * 1e3, reps * sample_bytes


def workload_text(wl, m: int, head: bool) -> str:
    return f"{wl.name}: {wl.description}, decode M={m}, {wl.layers} layers x 7 linears" + (" + lm_head" if head else "")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    n = max(1, args.steps)
    gbs, cores, sample, ms, _ = cpu_scheme_timing(wl, args.m, steps=n, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": max(1, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_text(wl, args.m, wl.head is not None and not args.no_head), "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference's quantized matmul scheme (candle-core is not vendored and no "
                "Rust toolchain exists here) on all host threads; each step is the bounded sample named in "
                "cpu_baseline.sample, value = its weight bytes per second",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU arm

GROUPS = [["attn_q", "attn_k", "attn_v"], ["attn_output"], ["ffn_gate", "ffn_up"], ["ffn_down"]]


class Stack:
    """The quantized linears of a workload resident on one GPU: every layer in buffers of its own,
    so a pass streams from HBM. gen = "oracle": seeded N(0, 0.02) weights through the CPU
    quantizer (host copies kept for the parity check); "device": seeded N(0, 0.02) weights
    quantized on the GPU by the library's weight quantizer (the secondary configurations)."""

    def __init__(self, wl, dev, gen="oracle", head=True, ctx=None):
        import torch
        from tur_b200 import GgmlDType, QMatMul, QTensor
        from tur_b200.workloads import quantized_blocks
        self.wl, self.dev, self.host_blocks = wl, dev, {}
        protos = []
        for i, w in enumerate(wl.per_layer):
            if gen == "oracle":
                hb = gen_weight_blocks(w, SEED + i)
                self.host_blocks[w.name] = hb
                protos.append((w, torch.from_numpy(hb).to(dev)))
            else:
                protos.append((w, quantized_blocks(w.dtype, w.n, w.k, SEED + i, dev)))
        self.layers = [[(w, QMatMul.from_arc(QTensor.new(b, GgmlDType(w.dtype), (w.n, w.k), ctx=ctx))) for w, b in protos]
                       for _ in range(wl.layers)]
        self.head = None
        if wl.head is not None and head:
            if gen == "oracle":
                hb = gen_weight_blocks(wl.head, SEED + 999)
                self.host_blocks[wl.head.name] = hb
                b = torch.from_numpy(hb).to(dev)
            else:
                b = quantized_blocks(wl.head.dtype, wl.head.n, wl.head.k, SEED + 999, dev)
            self.head = (wl.head, QMatMul.from_arc(QTensor.new(b, GgmlDType(wl.head.dtype), (wl.head.n, wl.head.k), ctx=ctx)))
        del protos
        torch.cuda.synchronize()

    def weights(self):
        return list(self.wl.per_layer) + ([self.wl.head] if self.head else [])

    def pass_bytes(self):
        return self.wl.layers * self.wl.layer_bytes() + (self.wl.head.nbytes if self.head else 0)

    def pass_flops(self, m):
        return m * (self.wl.layers * sum(2 * w.n * w.k for w in self.wl.per_layer)
                    + (2 * self.wl.head.n * self.wl.head.k if self.head else 0))

    def buffers(self, m, xdtype="f32", host=False):
        """Seeded activations per source and output buffers per weight: device tensors, or
        page-locked host tensors for the end-to-end arm."""
        import torch
        srcs = sorted({(w.source, w.k) for w in self.wl.per_layer})
        xs = {s: torch.from_numpy(gen_activations(m, k, SEED + 10**6 + m + j)) for j, (s, k) in enumerate(srcs)}
        if host:
            x = {s: t.pin_memory() for s, t in xs.items()}
            y = {w.name: torch.empty((m, w.n), dtype=torch.float32).pin_memory() for w in self.weights()}
        else:
            x = {s: (t.to(self.dev).to(torch.bfloat16) if xdtype == "bf16" else t.to(self.dev)) for s, t in xs.items()}
            y = {w.name: torch.empty((m, w.n), dtype=torch.float32, device=self.dev) for w in self.weights()}
        return x, y

    def make_pass(self, x, y, mode, multi=True):
        """One pass over every linear of the stack, issued as a caller integrating the library
        would: linears that read the same x (attn_q|k|v, ffn_gate|up) as one multi-weight call."""
        from tur_b200 import QMatMul

        def run():
            for layer in self.layers:
                by_name = {w.name: (w, mm) for w, mm in layer}
                for grp in GROUPS:
                    members = [by_name[n] for n in grp if n in by_name]
                    if len(members) > 1 and multi:
                        QMatMul.forward_multi([mm for _, mm in members], x[members[0][0].source], mode=mode,
                                              outs=[y[w.name] for w, _ in members])
                    else:
                        for w, mm in members:
                            mm.forward(x[w.source], mode=mode, out=y[w.name])
            if self.head:
                self.head[1].forward(x["hidden"], mode=mode, out=y[self.head[0].name])
        return run


def _make_host_pass(self, x, y, mode, multi=True, bound=True):
    """The pass on page-locked host buffers. bound: every group of linears sharing x is a
    tur_b200.HostCall created once (device aliases resolved, launches recorded), as a decoder
    that reuses its activation buffers token after token would hold them; a step then runs them
    in order. Otherwise (or for more than 64 rows / other schemes) per-call host entries."""
    from tur_b200 import HostCall, Mode
    if not bound or mode != Mode.INT8_ACT or next(iter(x.values())).shape[0] > 64:
        return self.make_pass(x, y, mode, multi=multi)
    calls = []
    for layer in self.layers:
        by_name = {w.name: (w, mm) for w, mm in layer}
        for grp in GROUPS:
            members = [by_name[n] for n in grp if n in by_name]
            groups = [members] if (len(members) > 1 and multi) else [[mem] for mem in members]
            for g in groups:
                calls.append(HostCall([mm for _, mm in g], x[g[0][0].source], [y[w.name] for w, _ in g]))
    if self.head:
        calls.append(HostCall([self.head[1]], x["hidden"], [y[self.head[0].name]]))
    self._bound_calls = calls

    def run():
        for c in calls:
            c.run()
    return run


Stack.make_host_pass = _make_host_pass


def graph_of(fn, dev, ctx, warm=3):
    """Warm-up runs (they also size the context's scratch), then the pass captured as one CUDA
    graph. Returns (graph, launches per pass)."""
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    l0 = ctx.launch_count()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    launches = ctx.launch_count() - l0
    for _ in range(warm):
        g.replay()
    torch.cuda.synchronize()
    return g, launches


def time_replays(g, steps):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def sampled_rows(n, count, rng):
    rows = {r for r in (0, 15, 16, n // 2, n - 17, n - 16, n - 1) if 0 <= r < n}
    while len(rows) < min(count, n):
        rows.add(int(rng.integers(0, n)))
    return np.array(sorted(rows))


def parity_of_pass(stack, x, y, mode_name, m):
    """Compares what the timed pass left in its output buffers (the last layer's results; every
    layer holds the same weights and reads the same x, so they are layer 0's too) with the CPU
    oracle of the same scheme on a sample of weight rows. Outside every timed region."""
    import oracle
    import torch
    from tur_b200 import Mode
    rng = np.random.default_rng(SEED + 7)
    worst, checked, cross = 0.0, [], 0.0
    if mode_name == "EXACT_F32":
        mode_name = "F64"
    for w in stack.weights():
        if w.name not in stack.host_blocks:
            continue
        rows = sampled_rows(w.n, 128, rng)
        wb = stack.host_blocks[w.name][rows]
        xh = x[w.source].float().cpu().numpy()
        got = y[w.name][:, torch.from_numpy(rows).to(stack.dev)].cpu().numpy()
        want = oracle.qmatmul(w.dtype, wb, len(rows), w.k, xh) if mode_name == "INT8_ACT" else oracle.matmul_f64(w.dtype, wb, len(rows), w.k, xh)
        err = oracle.rel_fro(got, want)
        worst = max(worst, err)
        checked.append(f"{w.name} {TYPE_NAMES[w.dtype]} {w.n}x{w.k}")
    # cross-scheme distance on layer 0 (what AUTO's switch between 16 and 17 rows would change)
    for w, mm in stack.layers[0]:
        if w.k % 64:
            continue
        a = mm.forward(x[w.source], mode=Mode.INT8_ACT)
        b = mm.forward(x[w.source], mode=Mode.TENSOR_CORE)
        cross = max(cross, oracle.rel_fro(a.cpu().numpy(), b.cpu().numpy()))
    return {"rel_fro_max": worst, "tolerance": 2e-3, "oracle": "cpu scheme (oracle.qmatmul)" if mode_name == "INT8_ACT" else "f64 dequantize-then-matmul",
            "rows_sampled_per_weight": 128, "checked": checked, "int8_vs_f16_scheme_rel_fro_max": cross}


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from tur_b200 import Mode, QMatMul, context

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl = WORKLOADS[args.workload]
    m = args.m
    mode = Mode[args.mode]
    ctx = context(local)
    peak, peak_kind = measured_peaks()
    tpeak, tkind = measured_tensor_peak()

    stack = Stack(wl, dev, gen="oracle", head=not args.no_head)
    x_dev, y_dev = stack.buffers(m, args.xdtype)
    one_pass_device = stack.make_pass(x_dev, y_dev, mode, multi=not args.no_multi)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graph, launches_per_step = graph_of(one_pass_device, dev, ctx, warm=max(3, args.warmup))
    sampler = ClockSampler(local)
    # ---- timed region: K graph replays, device timed
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    barrier()
    ms = e0.elapsed_time(e1)
    tensor_path = mode == Mode.TENSOR_CORE or (mode == Mode.AUTO and m > 16)
    parity = parity_of_pass(stack, x_dev, y_dev, "TENSOR_CORE" if tensor_path else ("INT8_ACT" if mode != Mode.EXACT_F32 else "EXACT_F32"), m) \
        if rank == 0 and not args.no_parity else None

    # ---- end to end through the host-buffer entries: page-locked host x in, page-locked host y
    # out, one call per group of linears that share x, a synchronize inside every call
    e2e_ms = None
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    if not args.no_e2e:
        x_host, y_host = stack.buffers(m, host=True)
        one_pass_host = stack.make_host_pass(x_host, y_host, mode, multi=not args.no_multi, bound=not args.no_bound)
        for _ in range(3):
            one_pass_host()
        barrier()
        with sampler:
            t0 = time.perf_counter()
            e0.record()
            for _ in range(e2e_steps):
                one_pass_host()
            e1.record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3
        barrier()
        e2e_ms = max(e0.elapsed_time(e1), wall)
        if rank == 0 and parity is not None and not tensor_path:
            # the host route must give what the device route gave
            parity["e2e_equals_device_route"] = all(torch.equal(y_host[w.name], y_dev[w.name].cpu()) for w in stack.weights())

    # ---- dominant launch, timed alone over the layers' distinct buffers: the group of linears
    # sharing one x that moves the most bytes (ffn_gate|up in the decoder stacks), issued exactly
    # as the pass issues it (one multi-weight launch unless --no-multi)
    dom_names = max(GROUPS, key=lambda g: sum(w.nbytes for w in wl.per_layer if w.name in g))
    dom_ws = [w for w in wl.per_layer if w.name in dom_names]
    dom = dom_ws[0]

    def dom_pass():
        for layer in stack.layers:
            members = [(w, mm) for w, mm in layer if w.name in dom_names]
            if len(members) > 1 and not args.no_multi:
                QMatMul.forward_multi([mm for _, mm in members], x_dev[dom.source], mode=mode, outs=[y_dev[w.name] for w, _ in members])
            else:
                for w, mm in members:
                    mm.forward(x_dev[w.source], mode=mode, out=y_dev[w.name])

    dg, dl = graph_of(dom_pass, dev, ctx)
    dom_launches = dl / len(stack.layers)
    # per group: the GEMV launch plus, where the activations are not quantized in the kernel,
    # their quantization launch; timed together. x is read once for the whole group.
    dom_us = time_replays(dg, 20) * 1e3 / len(stack.layers)
    x_es = 2 if args.xdtype == "bf16" else 4
    alg_bytes = sum(w.nbytes + m * w.n * 4 for w in dom_ws) + m * dom.k * x_es

    extras = {}
    if rank == 0 and args.workload == "cfg2" and m == 1 and not args.no_extras:
        extras = run_extras(stack, dev, ctx, peak, tpeak, local)

    pass_bytes, pass_flops = stack.pass_bytes(), stack.pass_flops(m)
    head_w = stack.head[0] if stack.head else None

    # ---- the sharded workload (cfg5) at this rank count: every rank takes part
    tp_obj = None
    if world > 1 and args.workload == "cfg2" and m == 1 and not args.no_extras:
        del graph, dg
        stack.layers, stack.head = [], None
        torch.cuda.empty_cache()
        tp_obj = tp_measure(WORKLOADS["cfg5"], dev, ctx, rank, world, [(1, "INT8_ACT", "f32"), (64, "AUTO", "f32")], steps=10)

    # ---- reduce over ranks
    if world > 1:
        t = torch.tensor([ms, e2e_ms or 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), (float(t[1]) if e2e_ms is not None else None)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    total_bytes = pass_bytes * world
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9
    achieved = alg_bytes / (dom_us * 1e-6) / 1e9
    traffic = NCU_TRAFFIC_BYTES.get((tuple(w.name for w in dom_ws), wl.name, m))
    grp_x = [max(w.k for w in wl.per_layer if w.name in g) for g in GROUPS]
    h2d = m * 4 * (sum(grp_x) * wl.layers + (head_w.k if head_w else 0))
    d2h = sum(m * w.n * 4 for w in wl.per_layer) * wl.layers + (m * head_w.n * 4 if head_w else 0)
    members = " | ".join(f"{w.name} {TYPE_NAMES[w.dtype]} {w.n}x{w.k}" for w in dom_ws)
    if tensor_path and m > 64:
        # prefill runs the tcgen05 GEMM: bound by the tensor cores (decode batches of up to 64 rows
        # stay bound by the weight stream whichever path computes them)
        dom_flops = 2.0 * m * sum(w.n * w.k for w in dom_ws)
        tf = dom_flops / (dom_us * 1e-6) / 1e12
        roofline = {"bound": "tensor", "kernel": "gemm_tc (+ activation prep) " + members + " as issued in the pass",
                    "achieved": tf, "peak": tpeak, "peak_kind": tkind, "unit": "TFLOP/s", "frac": tf / tpeak,
                    "us_per_launch": dom_us, "launches": dom_launches, "algorithmic_flops": dom_flops, "traffic": None}
    else:
        roofline = {"bound": "hbm",
                    "kernel": ("gemm_tc (+ activation prep, split-K reduction) " if tensor_path else "gemv_stream ") + members
                              + " as issued in the pass (one multi-weight launch where the path has one; activation "
                              "quantization included)",
                    "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                    "us_per_launch": dom_us, "launches": dom_launches, "algorithmic_bytes": alg_bytes, "traffic": traffic,
                    "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of this launch from one ncu capture"
                                    if traffic is not None else "no ncu capture of this launch"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("f16" if tensor_path else "int8" if mode in (Mode.INT8_ACT, Mode.AUTO) else "f32"), "data": "synthetic",
        "config": {
            "workload": workload_text(wl, m, head_w is not None),
            "mode": mode.name, "x_dtype": args.xdtype, "weight_bytes_per_step_per_gpu": pass_bytes,
            "tflops": pass_flops * world * args.steps / (ms * 1e-3) / 1e12, "parallelism": f"replicas x{world}",
            "l2": "weights per pass exceed L2 (distinct buffers per layer); CUDA-graph replay per step",
            "multi_weight_launch": not args.no_multi,
            "tokens_per_s": m * world * args.steps / (ms * 1e-3),
        },
        "e2e": None if e2e_ms is None else {
            "value": total_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "steps": e2e_steps,
            "ms_per_step": e2e_ms / e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "api": ("turq_host_call_run (calls bound once to their page-locked buffers)" if not args.no_bound and mode == Mode.INT8_ACT and m <= 64
                    else "turq_qmatmul_multi_host / turq_qmatmul_host") +
                   " per group of linears sharing x: page-locked host x in, page-locked host y out, one wait per "
                   "call (bound calls: on the completion word the call's last kernel stores into mapped host memory; others: a stream synchronize); the activation rows cross the bus once per call (read in place by the quantization launch), "
                   "every output once (written in place by the GEMV)"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": sampler.summary(),
        "roofline": roofline,
    }
    if parity is not None:
        line["parity"] = parity
    line.update(extras)
    if tp_obj is not None:
        line["tp"] = tp_obj
    if not args.no_cpu and world == 1:
        gbs, cores, sample, _, _ = cpu_scheme_timing(wl, m, steps=args.cpu_steps)
        line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_extras(stack, dev, ctx, peak, tpeak, local):
    """The other contract points of the benchmark configurations, measured in the same run with
    the weights already resident: the decode sweep M = 2..16, a prefill pass on the tensor cores,
    and the small / 3B stacks at M = 1. Each is a CUDA-graph replay timed with CUDA events."""
    import torch
    from tur_b200 import Mode
    out = {}
    wl = stack.wl
    sweep = []
    for mm_rows in (2, 4, 8, 16):
        x, y = stack.buffers(mm_rows)
        g, _ = graph_of(stack.make_pass(x, y, Mode.INT8_ACT), dev, ctx)
        t = time_replays(g, 10)
        gbs = stack.pass_bytes() / (t * 1e-3) / 1e9
        sweep.append({"rows": mm_rows, "ms_per_step": t, "weight_gbs": gbs, "frac_of_hbm_peak": gbs / peak,
                      "tokens_per_s": mm_rows / (t * 1e-3)})
        del g, x, y
    out["sweep"] = {"workload": f"{wl.name} decode, integer scheme, rows per pass 2..16 (same weights as the headline)", "points": sweep}
    # prefill: the same layers, no head (prefill evaluates it for one token), bf16 activations
    head, stack.head = stack.head, None
    try:
        pre = []
        for rows in (512, 2048):
            x, y = stack.buffers(rows, "bf16")
            sampler = ClockSampler(local)
            g, _ = graph_of(stack.make_pass(x, y, Mode.TENSOR_CORE), dev, ctx, warm=2)
            with sampler:
                t = time_replays(g, 5)
            tf = stack.pass_flops(rows) / (t * 1e-3) / 1e12
            sustained = None
            try:
                with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                    sustained = float(json.load(f)["bf16_tflops_sustained"])
            except Exception:
                pass
            pre.append({"rows": rows, "ms_per_step": t, "tflops": tf, "frac_of_burst_peak": tf / tpeak,
                        "frac_of_sustained_peak": (tf / sustained) if sustained else None, "clocks": sampler.summary()})
            del g, x, y
        out["prefill"] = {"workload": f"{wl.name} prefill, 36 layers x 7 linears, bf16 activations, tcgen05 f16 GEMM, no lm_head",
                          "points": pre}
    finally:
        stack.head = head
    torch.cuda.empty_cache()
    cfgs = []
    for name in ("cfg1", "cfg4-q5", "cfg4-q8"):
        st = Stack(WORKLOADS[name], dev, gen="device", head=False)
        x, y = st.buffers(1)
        g, launches = graph_of(st.make_pass(x, y, Mode.INT8_ACT), dev, ctx)
        t = time_replays(g, 10)
        gbs = st.pass_bytes() / (t * 1e-3) / 1e9
        cfgs.append({"workload": workload_text(st.wl, 1, False), "weights": "seeded N(0, 0.02) quantized on the GPU (turq_quantize_weights)",
                     "ms_per_step": t, "weight_gbs": gbs, "frac_of_hbm_peak": gbs / peak, "launches": launches})
        del g, x, y, st
        torch.cuda.empty_cache()
    out["configs"] = cfgs
    return out


class TPStack:
    """A workload's linears sharded Megatron-style over `world` ranks (this rank's shards only):
    attn_q|k|v by whole heads, ffn_gate|up in 256-row units and the head in 16-row units (rows:
    contiguous bytes), attn_output / ffn_down by whole blocks of columns. Weights are valid random
    blocks generated on the GPU, the same on every rank, sharded as bytes."""

    def __init__(self, wl, dev, rank, world, head=True, head_dim=128, layers=None):
        import torch
        from tur_b200 import GgmlDType, QMatMul, QTensor
        from tur_b200.tensor_parallel import row_unit_for, shard_blocks, shard_of, split_units
        from tur_b200.workloads import quantized_blocks
        self.wl, self.dev, self.rank, self.world = wl, dev, rank, world
        self.n_layers = layers or wl.layers

        def make(w, seed):
            sh = shard_of(w, world, rank, row_unit_for(w, head_dim))
            return sh, shard_blocks(quantized_blocks(w.dtype, w.n, w.k, seed, dev), w, sh).reshape(-1)

        protos = [(w,) + make(w, SEED + i) for i, w in enumerate(wl.per_layer)]
        self.layers = [[(w, sh, QMatMul.from_arc(QTensor.new(b, GgmlDType(w.dtype), sh.shape))) for w, sh, b in protos]
                       for _ in range(self.n_layers)]
        self.head = None
        if wl.head is not None and head:
            sh, b = make(wl.head, SEED + 999)
            self.head = (wl.head, sh, QMatMul.from_arc(QTensor.new(b, GgmlDType(wl.head.dtype), sh.shape)))
            self.head_widths = [c * 16 for _, c in split_units(wl.head.n // 16, world)]
        del protos
        torch.cuda.synchronize()

    def exchange_bytes(self, m):
        """Largest tensor any exchange of a pass moves (per rank for the gather)."""
        big = max(m * w.n * 4 for w, sh, _ in self.layers[0] if sh.parallel == "row")
        if self.head:
            big = max(big, m * max(self.head_widths) * 4)
        return big

    def buffers(self, m, xdtype="f32"):
        import torch
        xs, ys = {}, {}
        for w, sh, _ in self.layers[0]:
            kloc = sh.shape[1]
            if (w.source, kloc) not in xs:
                x = torch.from_numpy(gen_activations(m, kloc, SEED + 10**6 + m + len(xs))).to(self.dev)
                xs[(w.source, kloc)] = x.to(torch.bfloat16) if xdtype == "bf16" else x
            # row-parallel outputs are full width (summed over the ranks), column-parallel ones this rank's share
            ys[w.name] = torch.empty((m, sh.shape[0]), dtype=torch.float32, device=self.dev)
        if self.head:
            ys["output_local"] = torch.empty((m, self.head[1].shape[0]), dtype=torch.float32, device=self.dev)
            ys["output"] = torch.empty((m, self.wl.head.n), dtype=torch.float32, device=self.dev)
        return xs, ys

    def make_pass(self, xs, ys, mode, group=None):
        """group = a TPGroup: exchanges by the library's own kernels (graph-capturable);
        None: NCCL all-reduce / all-gather through torch.distributed (eager only)."""
        import torch.distributed as dist
        from tur_b200 import QMatMul
        from tur_b200.tensor_parallel import gather_columns
        world, wl = self.world, self.wl

        def run():
            for layer in self.layers:
                by_name = {w.name: (w, sh, mm) for w, sh, mm in layer}
                for grp in GROUPS:
                    same = [by_name[n] for n in grp]
                    w0, sh0, mm0 = same[0]
                    x = xs[(w0.source, sh0.shape[1])]
                    if len(same) > 1:
                        QMatMul.forward_multi([mm for _, _, mm in same], x, mode=mode, outs=[ys[w.name] for w, _, _ in same])
                    elif sh0.parallel == "row" and world > 1 and group is not None:
                        group.qmatmul_rowparallel(mm0, x, mode=mode, out=ys[w0.name])
                    else:
                        y = mm0.forward(x, mode=mode, out=ys[w0.name])
                        if sh0.parallel == "row" and world > 1:
                            dist.all_reduce(y)
            if self.head:
                if world > 1 and group is not None:
                    group.qmatmul_gather(self.head[2], xs[("hidden", wl.hidden)], self.head_widths, mode=mode, out=ys["output"])
                else:
                    y = self.head[2].forward(xs[("hidden", wl.hidden)], mode=mode, out=ys["output_local"])
                    if world > 1:
                        gather_columns(y, wl.head.n, world, 16)
        return run

    def collectives_per_pass(self):
        return sum(1 for w, sh, _ in self.layers[0] if sh.parallel == "row") * self.n_layers + (1 if self.head else 0)


def timed_max_over_ranks(fn, steps, dev, world):
    """`steps` calls of fn between barriers, device-timed, maximum over the ranks (ms per call)."""
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(t[0])


def tp_parity(stack, group, dev, ctx, m=4):
    """Sharded against unsharded on real ranks, layer 0's ffn_gate (column-parallel: gathered
    shares equal the unsharded product bit for bit when both launches deal out whole row-tiles,
    else within f32 reassociation) and ffn_down (row-parallel: summed partial products within f32
    reassociation)."""
    import torch
    from tur_b200 import GgmlDType, Mode, QMatMul, QTensor
    from tur_b200.tensor_parallel import split_units
    from tur_b200.workloads import quantized_blocks
    out = {}
    for i, (w, sh, mm) in enumerate(stack.layers[0]):
        if w.name not in ("ffn_gate", "ffn_down"):
            continue
        full = QMatMul.from_arc(QTensor.new(quantized_blocks(w.dtype, w.n, w.k, SEED + i, dev), GgmlDType(w.dtype), (w.n, w.k)))
        x = torch.from_numpy(gen_activations(m, w.k, SEED + 31 + i)).to(dev)
        ref = full.forward(x, mode=Mode.INT8_ACT)
        if sh.parallel == "column":
            widths = [c * sh.unit for _, c in split_units(w.n // sh.unit, stack.world)]
            got = group.allgather(mm.forward(x, mode=Mode.INT8_ACT), widths)
            # identical bits whenever shard and unsharded weight are both split in whole row-tiles;
            # a shard whose row-tiles get cut between CTAs adds its partial sums in another order
            out["column_parallel_bit_exact"] = bool(torch.equal(got, ref))
            out["column_parallel_rel_fro"] = float((got - ref).norm() / ref.norm())
        else:
            xl = x[:, sh.cols[0]: sh.cols[0] + sh.cols[1]].contiguous()
            got = group.qmatmul_rowparallel(mm, xl, mode=Mode.INT8_ACT)
            out["row_parallel_rel_fro"] = float((got - ref).norm() / ref.norm())
        del full
    ctx.poll_status()
    torch.cuda.empty_cache()
    return out


def tp_measure(wl, dev, ctx, rank, world, rows_modes, steps, head=True, own=True, one_gpu=True, fuse_limit=None,
               twoshot_limit=None, chunk_rows=None):
    """Strong scaling of one sharded pass: ms per pass at `world` ranks (CUDA-graph replay with the
    library's own exchange kernels when own=True, eager launches with NCCL collectives otherwise)
    and, measured by rank 0 alone in the same run, the unsharded pass on one GPU."""
    import torch
    import torch.distributed as dist
    from tur_b200 import Mode
    from tur_b200.tensor_parallel import TPGroup
    stack = TPStack(wl, dev, rank, world, head=head)
    group = None
    points, parity = [], None
    if own and world > 1:
        group = TPGroup(rank, world, max(stack.exchange_bytes(max(r for r, _, _ in rows_modes)), 4 * 25600 * 4), ctx=ctx)
        if fuse_limit is not None:
            group.set_fuse_limit(fuse_limit)
        if twoshot_limit is not None:
            group.set_twoshot_limit(twoshot_limit)
        if chunk_rows is not None:
            group.set_chunk_rows(chunk_rows)
        parity = tp_parity(stack, group, dev, ctx)
    for rows, mode_name, xdtype in rows_modes:
        mode = Mode[mode_name]
        xs, ys = stack.buffers(rows, xdtype)
        fn = stack.make_pass(xs, ys, mode, group)
        launches = None
        if own or world == 1:
            g, launches = graph_of(fn, dev, ctx)
            runner = g.replay
        else:
            for _ in range(3):
                fn()
            runner = fn
        ms = timed_max_over_ranks(runner, steps, dev, world)
        ctx.poll_status()
        points.append({"rows": rows, "mode": mode_name, "x_dtype": xdtype, "ms_per_step": ms, "launches_per_pass": launches,
                       "cuda_graph": bool(own or world == 1)})
        del xs, ys, fn, runner
    total_bytes = wl.layers * wl.layer_bytes() + (wl.head.nbytes if stack.head else 0)
    collectives = stack.collectives_per_pass()
    del stack
    torch.cuda.empty_cache()
    if one_gpu and world > 1:
        # the same pass, unsharded, on rank 0's GPU while the other ranks wait at the barrier
        if rank == 0:
            solo = TPStack(wl, dev, 0, 1, head=head)
            for pt, (rows, mode_name, xdtype) in zip(points, rows_modes):
                xs, ys = solo.buffers(rows, xdtype)
                g, _ = graph_of(solo.make_pass(xs, ys, Mode[mode_name], None), dev, ctx)
                pt["ms_per_step_1gpu"] = time_replays(g, max(3, steps // 2))
                pt["speedup_vs_1gpu"] = pt["ms_per_step_1gpu"] / pt["ms_per_step"]
                pt["strong_scaling_efficiency"] = pt["speedup_vs_1gpu"] / world
                del g, xs, ys
            del solo
            torch.cuda.empty_cache()
        dist.barrier()
    for pt in points:
        pt["weight_gbs_aggregate"] = total_bytes / (pt["ms_per_step"] * 1e-3) / 1e9
    return {"workload": f"{wl.name}: {wl.description}, tensor-parallel x{world}" + (" + lm_head" if head else ""),
            "weights": "seeded N(0, 0.02) quantized on the GPU (turq_quantize_weights), sharded as bytes",
            "exchange": ("own kernels over peer memory (turq_tp_*): all-reduce fused behind attn_output and ffn_down, "
                         "all-gather behind the head; no NCCL call inside the pass") if own else
                        "NCCL all-reduce after attn_output and ffn_down, all-gather after the head (eager launches)",
            "collectives_per_pass": collectives, "weight_bytes_total": total_bytes, "parity": parity, "points": points}


def run_gpu_tp(args):
    """Tensor-parallel pass of a sharded workload (cfg5) as the whole job: strong scaling, the
    model is fixed and every rank streams 1/N of it."""
    import torch
    import torch.distributed as dist
    from tur_b200 import Mode, context

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl = WORKLOADS[args.workload]
    m = args.m
    mode = Mode[args.mode]
    ctx = context(local)
    sampler = ClockSampler(local)
    with sampler:
        obj = tp_measure(wl, dev, ctx, rank, world, [(m, args.mode, args.xdtype)], args.steps, head=not args.no_head,
                         own=not args.nccl, one_gpu=not args.no_extras, fuse_limit=args.tp_fuse_limit,
                         twoshot_limit=args.tp_twoshot_limit, chunk_rows=args.tp_chunk_rows)
    if rank == 0:
        pt = obj["points"][0]
        ms = pt["ms_per_step"]
        total_bytes = obj["weight_bytes_total"]
        pass_flops = m * (wl.layers * sum(2 * w.n * w.k for w in wl.per_layer) + (0 if args.no_head else 2 * wl.head.n * wl.head.k))
        peak, peak_kind = measured_peaks()
        value = total_bytes / (ms * 1e-3) / 1e9
        tensor_path = mode == Mode.TENSOR_CORE or (mode == Mode.AUTO and m > 16)
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16" if tensor_path else "int8", "data": "synthetic",
            "config": {"workload": obj["workload"] + f", M={m}", "mode": mode.name,
                       "x_dtype": args.xdtype, "tflops": pass_flops / (ms * 1e-3) / 1e12,
                       "parallelism": f"tp{world}", "cuda_graph": pt["cuda_graph"], "exchange": obj["exchange"],
                       "collectives_per_pass": obj["collectives_per_pass"], "weights": obj["weights"],
                       "weight_bytes_total": total_bytes, "tokens_per_s": m / (ms * 1e-3)},
            "e2e": None, "gpu_launches": (pt["launches_per_pass"] or 0) * args.steps, "clocks": sampler.summary(),
            "tp": obj,
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None,
                         "kernel": "whole sharded pass per GPU (GEMV / GEMM kernels + exchanges)"},
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="turq", choices=["turq", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", dest="m", type=int, default=1, help="activation rows per linear (decode batch M)")
    ap.add_argument("--mode", default="INT8_ACT", choices=["AUTO", "INT8_ACT", "EXACT_F32", "TENSOR_CORE"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--cpu-steps", type=int, default=20, help="steps of about half a second each in the cpu_baseline leg")
    ap.add_argument("--tp", action="store_true", help="tensor-parallel over all ranks (the sharded cfg5 workload)")
    ap.add_argument("--tp-fuse-limit", type=int, default=None, help="tensor-parallel arm: largest result (bytes) exchanged inside the matmul kernel")
    ap.add_argument("--no-multi", action="store_true", help="one launch per weight (no q|k, gate|up multi-weight launches)")
    ap.add_argument("--no-bound", action="store_true", help="e2e arm: per-call host entries instead of bound host calls")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed pass's outputs")
    ap.add_argument("--tp-twoshot-limit", type=int, default=None, help="tensor-parallel arm: smallest result (bytes) exchanged as "
                    "reduce-scatter + gather")
    ap.add_argument("--tp-chunk-rows", type=int, default=None, help="tensor-parallel arm: rows per chunk of a prefill-sized row-parallel "
                    "product (its exchange overlaps the next chunk)")
    ap.add_argument("--no-extras", action="store_true", help="skip the sweep / prefill / other-config objects of the default run")
    ap.add_argument("--nccl", action="store_true", help="tensor-parallel arm: NCCL collectives and eager launches instead of the "
                                                      "library's own exchange kernels in a CUDA graph (prefill-sized exchanges)")
    ap.add_argument("--xdtype", default="f32", choices=["f32", "bf16"], help="activation dtype on the device (prefill configs use bf16)")
    ap.add_argument("--no-head", action="store_true", help="leave the lm_head out of the pass (prefill evaluates it for one token only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.tp:
        run_gpu_tp(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
