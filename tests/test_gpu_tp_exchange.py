"""The library's own tensor-parallel exchange (turq_tp_*) on ONE GPU: the other ranks are local
stand-ins whose part the host plays between calls, so no kernel ever waits for another kernel.
Checks the arithmetic and order of the reduction, the slot alternation over consecutive calls,
the fused row-parallel GEMV, graph replay, and that a peer that never arrives ends the wait with
TURQ_E_TIMEOUT while the context stays usable. Real multi-GPU runs are in test_tp_multi_gpu.py."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
SEED = 299792458


@pytest.fixture(scope="module")
def tq():
    from tur_b200 import quantized
    assert torch.cuda.is_available()
    return quantized


def test_single_rank_group_is_the_plain_matmul_and_replays_in_a_graph(tq):
    from tur_b200.tensor_parallel import TPGroup
    n, k, m = 320, 1024, 3
    rng = np.random.default_rng(SEED)
    w = oracle.quantize(oracle.Q4_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType.Q4K, (n, k)))
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    g = TPGroup(0, 1, m * n * 4)
    want = mm.forward(x, bias=bias, mode=tq.Mode.INT8_ACT)
    for _ in range(3):                                       # consecutive calls alternate the exchange slot
        assert torch.equal(g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.INT8_ACT), want)
    xs = x[:, :n].contiguous()                               # a slot holds m * n floats
    assert torch.equal(g.allreduce(xs), xs)
    assert torch.equal(g.allgather(xs, [n]), xs)
    # tensor-core scheme goes through the staging copy
    x64 = torch.from_numpy(rng.standard_normal((40, k)).astype(np.float32)).cuda()
    g2 = TPGroup(0, 1, 40 * n * 4)
    assert torch.equal(g2.qmatmul_rowparallel(mm, x64, mode=tq.Mode.TENSOR_CORE), mm.forward(x64, mode=tq.Mode.TENSOR_CORE))
    # a captured graph replays the same launches: the call number lives on the device
    out = torch.empty((m, n), device="cuda")
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.INT8_ACT, out=out)
        g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.INT8_ACT, out=out)
        g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.INT8_ACT, out=out)   # odd count: replays start on alternating slots
    for _ in range(4):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    tq.context().poll_status()
    with pytest.raises(tq.TurqError) as e:
        g.allreduce(torch.zeros(m * n + 4, device="cuda"))   # more than the slot holds
    assert e.value.status == 9


@pytest.mark.parametrize("world,rank", [(2, 0), (4, 2), (8, 7)])
def test_reduction_adds_the_ranks_in_rank_order(tq, world, rank):
    from tur_b200.tensor_parallel import TPGroup
    n, k, m = 528, 512, 5
    rng = np.random.default_rng(SEED + world)
    w = oracle.quantize(oracle.Q6_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType.Q6K, (n, k)))
    g = TPGroup(rank, world, m * n * 4, loopback=True)
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    for call in range(3):
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
        own = mm.forward(x, mode=tq.Mode.INT8_ACT)
        parts = [torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).cuda() for _ in range(world)]
        parts[rank] = own
        for p in range(world):
            if p != rank:
                g.loopback_fill(p, parts[p], signal=True)     # the stand-in "peer" has written its slot and signalled
        y = g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.INT8_ACT)
        want = parts[0].clone()
        for p in range(1, world):
            want += parts[p]                                  # rank order, one rounding per addition
        want += bias
        assert torch.equal(y, want), call
    # all-gather with uneven widths
    widths = [16 * (3 + (p % 3)) for p in range(world)]
    shares = [torch.from_numpy(rng.standard_normal((m, wd)).astype(np.float32)).cuda() for wd in widths]
    for p in range(world):
        if p != rank:
            g.loopback_fill(p, shares[p], signal=True)
    assert torch.equal(g.allgather(shares[rank], widths), torch.cat(shares, dim=1))
    # the head's product gathered in one call: this rank's columns come from its matmul
    widths2 = [n if p == rank else 16 * (2 + p) for p in range(world)]
    shares2 = [torch.from_numpy(rng.standard_normal((m, wd)).astype(np.float32)).cuda() for wd in widths2]
    shares2[rank] = mm.forward(x, bias=bias, mode=tq.Mode.INT8_ACT)
    for p in range(world):
        if p != rank:
            g.loopback_fill(p, shares2[p], signal=True)
    assert torch.equal(g.qmatmul_gather(mm, x, widths2, bias=bias, mode=tq.Mode.INT8_ACT), torch.cat(shares2, dim=1))
    # a result larger than the fused limit takes the separate exchange launch: same arithmetic
    big_m = 40                                                 # 40 x 528 x 4 B = 84 KB > 64 KB
    xb = torch.from_numpy(rng.standard_normal((big_m, k)).astype(np.float32)).cuda()
    gb = TPGroup(rank, world, big_m * n * 4, loopback=True)
    parts = [torch.from_numpy(rng.standard_normal((big_m, n)).astype(np.float32)).cuda() for _ in range(world)]
    parts[rank] = mm.forward(xb, mode=tq.Mode.INT8_ACT)
    for p in range(world):
        if p != rank:
            gb.loopback_fill(p, parts[p], signal=True)
    want = parts[0].clone()
    for p in range(1, world):
        want += parts[p]
    assert torch.equal(gb.qmatmul_rowparallel(mm, xb, mode=tq.Mode.INT8_ACT), want)
    tq.context().poll_status()


@pytest.mark.parametrize("world,rank", [(4, 1), (8, 7), (3, 0)])
def test_two_shot_exchange_reduces_one_slice_and_copies_the_others(tq, world, rank):
    """Large results on three or more ranks: this rank adds its slice of the float4 groups in rank
    order and takes the other slices, already reduced, from their owners. The stand-ins hold what
    a real peer's slot holds at the second meeting point: its partial, with its own slice replaced
    by the reduced values."""
    from tur_b200.tensor_parallel import TPGroup
    rng = np.random.default_rng(SEED + 17 * world)
    count = 4 * 5000 + 4 * world - 4          # slices of unequal length at the end
    g = TPGroup(rank, world, count * 4, loopback=True)
    g.set_twoshot_limit(1)
    nvec = count // 4
    per = (nvec + world - 1) // world
    for call in range(3):
        parts = [torch.from_numpy(rng.standard_normal(count).astype(np.float32)).cuda() for _ in range(world)]
        want = parts[0].clone()
        for p in range(1, world):
            want += parts[p]
        for p in range(world):
            if p == rank:
                continue
            slot = parts[p].clone()
            lo, hi = 4 * p * per, min(4 * (p + 1) * per, count)
            slot[lo:hi] = want[lo:hi]
            g.loopback_fill(p, slot, signal=True)
        assert torch.equal(g.allreduce(parts[rank]), want), call
    tq.context().poll_status()


def test_prefill_sized_row_parallel_product_is_cut_into_chunks(tq):
    """Chunks of rows whose exchange runs on the group's second stream while the next chunk is
    computed. One GPU: the stand-in peer contributes zeros and has arrived at every chunk's
    meeting point ahead of time, so the result is this rank's own product - the same bits as the
    plain matmul - eager and in a replayed graph."""
    from tur_b200.tensor_parallel import TPGroup
    n, k, m = 512, 1024, 1024 + 128
    rng = np.random.default_rng(SEED + 4321)
    w = oracle.quantize(oracle.Q4_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType.Q4K, (n, k)))
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    want = mm.forward(x, bias=bias, mode=tq.Mode.TENSOR_CORE)
    g = TPGroup(0, 2, 256 * n * 4, loopback=True)      # a slot holds one chunk, not the product
    g.set_chunk_rows(256)                              # 5 chunks (the last one 128 rows)
    g.loopback_fill(1, None, signal=40)
    y = g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.TENSOR_CORE)
    assert torch.equal(y, want)
    out = torch.empty_like(y)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        g.qmatmul_rowparallel(mm, x, bias=bias, mode=tq.Mode.TENSOR_CORE, out=out)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    tq.context().poll_status()


@pytest.mark.parametrize("m", [40, 300], ids=["split_k_reduction_picks_the_slot", "gemm_epilogue_picks_the_slot"])
def test_tensor_core_product_lands_in_the_exchange_slot_without_a_copy(tq, m):
    """In the tensor-core mode the GEMM's epilogue (or, for decode batches, its split-K
    reduction) reads the call counter on the device and writes the slot of the upcoming call
    itself. Four calls in a row alternate the slots; the stand-in peer contributes fresh data to
    each, so a product written to the wrong slot would show."""
    from tur_b200.tensor_parallel import TPGroup
    n, k = 384, 1024
    rng = np.random.default_rng(SEED + 99 + m)
    w = oracle.quantize(oracle.Q6_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType.Q6K, (n, k)))
    g = TPGroup(0, 2, m * n * 4, loopback=True)
    for call in range(4):
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
        peer = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).cuda()
        g.loopback_fill(1, peer, signal=True)
        y = g.qmatmul_rowparallel(mm, x, mode=tq.Mode.TENSOR_CORE)
        assert torch.equal(y, mm.forward(x, mode=tq.Mode.TENSOR_CORE) + peer), call
    tq.context().poll_status()


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status(tq):
    from tur_b200.tensor_parallel import TPGroup
    ctx = tq.new_context()
    g = TPGroup(0, 2, 4096, ctx=ctx, loopback=True)
    g.set_wait_limit(2_000_000)                               # about a millisecond of SM clock
    x = torch.ones(1024, device="cuda")
    out = torch.full_like(x, -1.0)
    g.allreduce(x, out=out)                                   # rank 1 never signals
    with pytest.raises(tq.TurqError) as e:
        ctx.poll_status()
    assert e.value.status == 7
    assert torch.equal(out, torch.full_like(x, -1.0))         # the exchange was skipped, nothing half-written
    ctx.poll_status()                                         # status cleared, context usable
    g.reset()
    g.loopback_fill(1, torch.full_like(x, 2.0), signal=True)
    assert torch.equal(g.allreduce(x), torch.full_like(x, 3.0))
    ctx.poll_status()
