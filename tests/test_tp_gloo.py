"""Tensor-parallel host logic on CPU: partition arithmetic, byte-level sharding of GGUF
blocks, and the collective pattern (all-reduce after row-parallel linears, all-gather after
column-parallel ones) with two gloo ranks. The per-rank product is the CPU oracle here; on a
GPU it is tur_b200.QMatMul (tests/test_gpu_parity.py covers shard reassembly there)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tur_b200.tensor_parallel import TPLinear, gather_columns, row_unit_for, shard_blocks, shard_of, split_units
from tur_b200.workloads import WORKLOADS, Q4_K, Q6_K, Q8_0, Weight


def test_split_units_is_contiguous_and_balanced():
    assert [c for _, c in split_units(100, 8)] == [13, 13, 13, 13, 12, 12, 12, 12]
    parts = split_units(37, 5)
    assert parts[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(parts, parts[1:]))
    assert sum(c for _, c in parts) == 37
    with pytest.raises(ValueError):
        split_units(3, 4)


def test_qwen3_32b_partition_at_tp8_matches_the_block_structure():
    wl = WORKLOADS["cfg5"]
    by = {w.name: w for w in wl.per_layer}
    gate = [shard_of(by["ffn_gate"], 8, r, row_unit_for(by["ffn_gate"])).shape[0] for r in range(8)]
    down = [shard_of(by["ffn_down"], 8, r, row_unit_for(by["ffn_down"])).shape[1] for r in range(8)]
    assert gate == [3328] * 4 + [3072] * 4 and down == gate       # 25600 = 100 super-blocks: 13,13,13,13,12,12,12,12
    q = [shard_of(by["attn_q"], 8, r, 128).shape[0] for r in range(8)]
    o = [shard_of(by["attn_output"], 8, r, 128).shape[1] for r in range(8)]
    kv = [shard_of(by["attn_k"], 8, r, 128).shape[0] for r in range(8)]
    assert q == [1024] * 8 and o == q and kv == [128] * 8          # 64 q heads, 8 kv heads of 128
    head = [shard_of(wl.head, 8, r).shape[0] for r in range(8)]
    assert sum(head) == 151936 and max(head) - min(head) <= 16


@pytest.mark.parametrize("dt", [Q8_0, Q4_K, Q6_K])
def test_shard_bytes_dequantize_to_the_matching_slice(dt):
    rng = np.random.default_rng(5)
    n, k = 48, 1024
    w = Weight("ffn_down", n, k, dt, "inter", "row")
    blocks = oracle.quantize(dt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    full = oracle.dequantize(dt, blocks, k)
    for tp in (2, 3):
        for r in range(tp):
            sh = shard_of(w, tp, r, 256)
            part = oracle.dequantize(dt, shard_blocks(blocks, w, sh), sh.shape[1])
            assert np.array_equal(part, full[:, sh.cols[0]: sh.cols[0] + sh.cols[1]])
    wc = Weight("attn_q", n, k, dt, "hidden", "column")
    for r in range(3):
        sh = shard_of(wc, 3, r, 16)
        part = oracle.dequantize(dt, shard_blocks(blocks, wc, sh), k)
        assert np.array_equal(part, full[sh.rows[0]: sh.rows[0] + sh.rows[1]])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        rng = np.random.default_rng(11)          # same stream on every rank: same full weights
        hidden, inter, m = 512, 768, 3
        gate = Weight("ffn_gate", inter, hidden, Q4_K, "hidden", "column")
        down = Weight("ffn_down", hidden, inter, Q6_K, "inter", "row")
        gb = oracle.quantize(Q4_K, (rng.standard_normal((inter, hidden)) * 0.02).astype(np.float32))
        db = oracle.quantize(Q6_K, (rng.standard_normal((hidden, inter)) * 0.02).astype(np.float32))
        x = rng.standard_normal((m, hidden)).astype(np.float32)

        def cpu_matmul(w, blocks, sh):
            sb = shard_blocks(blocks, w, sh)
            return lambda t: torch.from_numpy(oracle.matmul_f64(w.dtype, sb, sh.shape[0], sh.shape[1], t.numpy()))

        gsh, dsh = shard_of(gate, world, rank, 256), shard_of(down, world, rank, 256)
        g = TPLinear(gate, gsh, cpu_matmul(gate, gb, gsh))
        d = TPLinear(down, dsh, cpu_matmul(down, db, dsh))
        h_local = g(torch.from_numpy(x))                      # [m, inter / world]: this rank's columns
        assert h_local.shape == (m, gsh.shape[0])
        h_full = gather_columns(h_local, inter, world, 256)   # what a vocab-sharded head would do
        want_h = oracle.matmul_f64(Q4_K, gb, inter, hidden, x)
        assert np.array_equal(h_full.numpy(), want_h)          # column-parallel pieces are exact
        y = d(h_local.contiguous())                           # row-parallel + all-reduce
        want_y = oracle.matmul_f64(Q6_K, db, hidden, inter, want_h)
        err = oracle.rel_fro(y.numpy(), want_y)
        assert err < 1e-5, err
        # an attention projection split by whole heads of 80 rows, three heads on two ranks (2 + 1):
        # the gather inside TPLinear must use the shard's own unit, not a fixed 16
        attn_q = Weight("attn_q", 240, hidden, Q4_K, "hidden", "column")
        qb = oracle.quantize(Q4_K, (rng.standard_normal((240, hidden)) * 0.02).astype(np.float32))
        qsh = shard_of(attn_q, world, rank, row_unit_for(attn_q, 80))
        assert qsh.unit == 80 and qsh.shape[0] == (160 if rank == 0 else 80)
        q_full = TPLinear(attn_q, qsh, cpu_matmul(attn_q, qb, qsh), gather_output=True)(torch.from_numpy(x))
        assert np.array_equal(q_full.numpy(), oracle.matmul_f64(Q4_K, qb, 240, hidden, x))
        # every rank ends with the same, complete result
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        assert all(torch.equal(ys[0], t) for t in ys)
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put((rank, repr(e)))


def test_two_gloo_ranks_reproduce_the_unsharded_mlp():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
