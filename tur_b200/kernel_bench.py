"""Per-kernel timing of the quantized-linear kernels on one GPU.

  python -m tur_b200.kernel_bench --op qmatmul --dtype Q4_K --n 12288 --k 4096 --m 1

Rotates through `--copies` distinct weight buffers (default: enough to exceed L2 several
times) so every launch streams from HBM, times `--iters` rounds with CUDA events on the
launching stream and prints one JSON line with the average time per call, the algorithmic
bytes (GGUF weight bytes + activations + outputs) and the implied bandwidth / flop rate.
Small `--copies/--iters` values make it a suitable target for an `ncu` capture.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import GgmlDType, Mode, QMatMul, QTensor, context
from .workloads import BLOCK, SEED, random_blocks

NAMES = {"Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="qmatmul", choices=["qmatmul", "dequantize", "embedding"])
    ap.add_argument("--dtype", default="Q4_K", choices=sorted(NAMES))
    ap.add_argument("--n", type=int, default=12288)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--mode", default="INT8_ACT", choices=["AUTO", "INT8_ACT", "EXACT_F32", "TENSOR_CORE"])
    ap.add_argument("--xdtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--pair", action="store_true", help="qmatmul: two weights of this shape that share x as ONE multi-weight "
                                                        "launch (how a decoder pass issues ffn_gate|up)")
    args = ap.parse_args()

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dt = NAMES[args.dtype]
    be, bb = BLOCK[dt]
    wbytes = args.n * (args.k // be) * bb
    copies = args.copies or max(2, min(64, int(4 * 126e6 / wbytes) + 1))
    if args.pair:
        copies = 2 * ((copies + 1) // 2)
    ws = []
    for i in range(copies):
        blocks = random_blocks(dt, args.n, args.k, SEED + i, dev)
        ws.append(QMatMul.from_arc(QTensor.new(blocks, GgmlDType(dt), (args.n, args.k))))
        del blocks
    rng = np.random.default_rng(SEED + 10**6 + args.m)
    x = torch.from_numpy(rng.standard_normal((args.m, args.k), dtype=np.float32)).to(dev)
    if args.xdtype == "bf16":
        x = x.to(torch.bfloat16)
    mode = Mode[args.mode]
    ctx = context(0)
    if args.op == "qmatmul":
        y = torch.empty((args.m, args.n), dtype=torch.float32, device=dev)

        y2 = torch.empty_like(y)

        def call(w):
            w.forward(x, mode=mode, out=y)
        alg_bytes = wbytes + args.m * args.k * x.element_size() + args.m * args.n * 4
        if args.pair:
            alg_bytes = 2 * (wbytes + args.m * args.n * 4) + args.m * args.k * x.element_size()
        flops = 2.0 * args.m * args.n * args.k
    elif args.op == "embedding":
        # --m ids drawn from the table's rows; algorithmic bytes = the rows read + the f32 rows written
        ids = torch.from_numpy(rng.integers(0, args.n, size=args.m)).to(dev).to(torch.int32)
        out = torch.empty((args.m, args.k), dtype=torch.float32, device=dev)

        def call(w):
            ctx.check(__import__("tur_b200")._lib.load().turq_embedding(
                ctx.handle, w.qtensor._h, ids.data_ptr(), args.m, 0, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
        alg_bytes = args.m * (args.k // be) * bb + args.m * args.k * 4
        flops = 0.0
    else:
        out = torch.empty((args.n, args.k), dtype=torch.float32, device=dev)

        def call(w):
            ctx.check(__import__("tur_b200")._lib.load().turq_dequantize(
                ctx.handle, w.qtensor._h, 0, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
        alg_bytes = wbytes + args.n * args.k * 4
        flops = 0.0

    def one_round():
        if args.pair and args.op == "qmatmul":
            for a, b in zip(ws[0::2], ws[1::2]):
                QMatMul.forward_multi([a, b], x, mode=mode, outs=[y, y2])
            return
        for w in ws:
            call(w)

    for _ in range(args.warmup):
        one_round()
    torch.cuda.synchronize()
    l0 = ctx.launch_count()
    runner = one_round
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
            one_round()
        runner = graph.replay
        runner()
    launches_per_call = (ctx.launch_count() - l0) / (copies // 2 if (args.pair and args.op == "qmatmul") else copies) if not args.no_graph else None
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        runner()
    e1.record()
    torch.cuda.synchronize()
    calls = copies // 2 if (args.pair and args.op == "qmatmul") else copies
    us = e0.elapsed_time(e1) * 1e3 / (args.iters * calls)
    if args.pair and args.op == "qmatmul":
        wbytes, flops = 2 * wbytes, 2 * flops
    print(json.dumps({
        "op": args.op, "dtype": args.dtype, "n": args.n, "k": args.k, "m": args.m, "mode": args.mode,
        "copies": copies, "pair": bool(args.pair), "iters": args.iters, "us_per_call": us, "launches_per_call": launches_per_call,
        "algorithmic_bytes": alg_bytes, "GBps": alg_bytes / us / 1e3, "weight_GBps": wbytes / us / 1e3,
        "TFLOPs": flops / us / 1e6,
    }))


if __name__ == "__main__":
    main()
