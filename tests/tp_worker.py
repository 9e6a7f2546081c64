"""One rank of the multi-GPU exchange test (launched by test_tp_multi_gpu.py through
torch.distributed.run, one process per GPU). Prints "TP_WORKER_OK <rank>" when every check passed.

Checks, on real peers: the library's all-reduce adds the ranks' tensors in rank order (bit-exact
against an explicit ordered sum of all-gathered inputs), its all-gather places uneven shares,
column-parallel shards reassemble the unsharded product bit for bit, row-parallel shards within
f32 reassociation, and a CUDA graph holding exchanges replays correctly many times."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    from tur_b200 import GgmlDType, Mode, QMatMul, QTensor, context
    from tur_b200.tensor_parallel import TPGroup, shard_blocks, shard_of, split_units
    from tur_b200.workloads import Q4_K, Q6_K, Weight, random_blocks

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = context(local)
    m = 5
    down = Weight("ffn_down", 1024, 256 * 13, Q6_K, "inter", "row")       # 13 blocks: uneven split
    gate = Weight("ffn_gate", 256 * 11, 1024, Q4_K, "hidden", "column")   # 11 units of 256 rows: uneven split
    g = TPGroup(rank, world, max(m * down.n, m * gate.n) * 4, ctx=ctx)

    # ---- all-reduce: bit-exact against the ordered sum
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    for count in (4, 1000, 5120, 65536 + 3):
        if count * 4 > max(m * down.n, m * gate.n) * 4:
            continue
        x = torch.randn(count, device=dev, generator=gen)
        everyone = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(everyone, x)
        want = everyone[0].clone()
        for p in range(1, world):
            want += everyone[p]
        got = g.allreduce(x)
        assert torch.equal(got, want), f"allreduce count={count}"

    # ---- sharded linears against the unsharded ones on this GPU (same bytes on every rank)
    for w in (down, gate):
        full_blocks = random_blocks(w.dtype, w.n, w.k, 77 + w.n, dev)
        full = QMatMul.from_arc(QTensor.new(full_blocks, GgmlDType(w.dtype), (w.n, w.k)))
        sh = shard_of(w, world, rank, 256)
        mine = QMatMul.from_arc(QTensor.new(shard_blocks(full_blocks, w, sh).reshape(-1), GgmlDType(w.dtype), sh.shape))
        x = torch.from_numpy(np.random.default_rng(5).standard_normal((m, w.k)).astype(np.float32)).to(dev)
        ref = full.forward(x, mode=Mode.INT8_ACT)
        if w.parallel == "row":
            xl = x[:, sh.cols[0]: sh.cols[0] + sh.cols[1]].contiguous()
            y = g.qmatmul_rowparallel(mine, xl, mode=Mode.INT8_ACT)
            err = float((y - ref).norm() / ref.norm())
            assert err < 1e-5, f"row-parallel rel error {err}"
            # every rank holds the same bits
            everyone = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(everyone, y)
            assert all(torch.equal(everyone[0], e) for e in everyone)
            # and a graph of several exchanges replays
            out = torch.empty_like(y)
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
                for _ in range(3):
                    g.qmatmul_rowparallel(mine, xl, mode=Mode.INT8_ACT, out=out)
            dist.barrier()
            for _ in range(20):
                graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, y), "graph replay"
        else:
            yl = mine.forward(x, mode=Mode.INT8_ACT)
            widths = [c * 256 for _, c in split_units(w.n // 256, world)]
            y = g.allgather(yl, widths)
            assert torch.equal(y, ref), "column-parallel gather"
            assert torch.equal(g.qmatmul_gather(mine, x, widths, mode=Mode.INT8_ACT), ref), "gather fused behind the matmul"
    # ---- large results: the two-shot exchange on three or more ranks (one-shot on two), bit-exact
    # against the ordered sum, identical on every rank; then a prefill-sized row-parallel product
    # cut into chunks whose exchanges overlap the next chunk's GEMM, eager and as a graph
    big = TPGroup(rank, world, ((1 << 20) + 256) * 4, ctx=ctx)
    big.set_twoshot_limit(1 << 20)                     # both sizes below take the two-shot form on 3+ ranks
    for count in (1 << 18, (1 << 20) + 4 * 37):
        x = torch.randn(count, device=dev, generator=gen)
        everyone = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(everyone, x)
        want = everyone[0].clone()
        for p in range(1, world):
            want += everyone[p]
        got = big.allreduce(x)
        assert torch.equal(got, want), f"large allreduce count={count}"
    w = down
    full_blocks = random_blocks(w.dtype, w.n, w.k, 77 + w.n, dev)
    sh = shard_of(w, world, rank, 256)
    full = QMatMul.from_arc(QTensor.new(full_blocks, GgmlDType(w.dtype), (w.n, w.k)))
    mine = QMatMul.from_arc(QTensor.new(shard_blocks(full_blocks, w, sh).reshape(-1), GgmlDType(w.dtype), sh.shape))
    mp = 1536
    xp = torch.from_numpy(np.random.default_rng(6).standard_normal((mp, w.k)).astype(np.float32)).to(dev).to(torch.bfloat16)
    xl = xp[:, sh.cols[0]: sh.cols[0] + sh.cols[1]].contiguous()
    ref = full.forward(xp, mode=Mode.TENSOR_CORE)
    whole = TPGroup(rank, world, mp * down.n * 4, ctx=ctx)
    whole.set_chunk_rows(1 << 20)                      # never cut: the unchunked exchange of the same product
    y_whole = whole.qmatmul_rowparallel(mine, xl, mode=Mode.TENSOR_CORE)
    big.set_chunk_rows(256)                            # 6 chunks
    y = big.qmatmul_rowparallel(mine, xl, mode=Mode.TENSOR_CORE)
    err = float((y - ref).norm() / ref.norm())
    assert err < 2e-3, f"chunked row-parallel rel error {err}"
    assert torch.equal(y, y_whole), "chunked and unchunked exchange disagree"
    everyone = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(everyone, y)
    assert all(torch.equal(everyone[0], e) for e in everyone)
    out = torch.empty_like(y)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        big.qmatmul_rowparallel(mine, xl, mode=Mode.TENSOR_CORE, out=out)
    dist.barrier()
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, y), "graph replay of the chunked product"
    ctx.poll_status()
    dist.barrier()
    whole.close()
    big.close()
    g.close()
    dist.destroy_process_group()
    print(f"TP_WORKER_OK {rank}", flush=True)


if __name__ == "__main__":
    main()
