"""Parity at the shapes the benchmark configurations name (Qwen3-8B / 3B / Qwen3-32B linears and
the 151936-row lm_head), where tile indices, grid sizes and split-K shares are far from the small
cases: the CUDA path against the CPU oracle on a sample of weight rows.

Weights are valid random blocks generated on the GPU (the CPU quantizer would take minutes for
these sizes); parity is defined on the bytes, so only the sampled rows' blocks go to the host.
Every weight row is an independent run of blocks, so the oracle's result for a subset of rows
equals those columns of the full product."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
SEED = 299792458
TOL = 2e-3
Q8_0, Q4_K, Q5_K, Q6_K = oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K


@pytest.fixture(scope="module")
def tq():
    from tur_b200 import quantized
    assert torch.cuda.is_available()
    return quantized


def sample_rows(n, count, rng):
    """First and last rows, both sides of 16-row tile and 128-row GEMM-tile borders, and random ones."""
    fixed = [0, 1, 15, 16, 17, 127, 128, n // 2, n - 129, n - 128, n - 17, n - 16, n - 2, n - 1]
    rows = {r for r in fixed if 0 <= r < n}
    while len(rows) < min(count, n):
        rows.add(int(rng.integers(0, n)))
    return np.array(sorted(rows))


def make(tq, dt, n, k, seed):
    from tur_b200.workloads import BLOCK, random_blocks
    dev = torch.device("cuda", torch.cuda.current_device())
    blocks = random_blocks(dt, n, k, seed, dev)
    qt = tq.QTensor.new(blocks, tq.GgmlDType(dt), (n, k))
    be, bb = BLOCK[dt]
    return qt, blocks.reshape(n, (k // be) * bb)


def check_int8(tq, qt, blocks2d, dt, n, k, x, y, rows):
    w = blocks2d[torch.from_numpy(rows).to(blocks2d.device)].cpu().numpy()
    want = oracle.qmatmul(dt, w, len(rows), k, x)
    got = y[:, torch.from_numpy(rows).to(y.device)].cpu().numpy()
    err = oracle.rel_fro(got, want)
    assert err < 1e-5, err           # same scheme: only the f32 summation order differs
    assert np.isfinite(y.float().sum().item())


@pytest.mark.parametrize("dt,n,k,ms", [
    (Q6_K, 151936, 4096, (1, 16)),     # cfg2 lm_head: 2.4 M tiles
    (Q6_K, 49155, 2560, (1, 5)),       # cfg4 head: ragged last row-tile, rows of 2100 bytes
    (Q8_0, 49155, 2560, (1, 5)),
    (Q6_K, 5120, 25600, (1, 8)),       # cfg5 ffn_down: rows of 21000 bytes, 100 tiles per row
    (Q4_K, 25600, 5120, (1, 8)),       # cfg5 ffn_gate
    (Q5_K, 8192, 2560, (1, 32)),       # cfg4 ffn_gate, decode batch 32 (planes read from global memory)
], ids=["lm_head_151936x4096_q6k", "head_49155x2560_q6k", "head_49155x2560_q8_0", "down_5120x25600_q6k",
        "gate_25600x5120_q4k", "gate_8192x2560_q5k"])
def test_integer_scheme_at_config_shapes(tq, dt, n, k, ms):
    rng = np.random.default_rng(SEED + n + k)
    qt, blocks2d = make(tq, dt, n, k, SEED + n)
    mm = tq.QMatMul.from_arc(qt)
    rows = sample_rows(n, 256, rng)
    for m in ms:
        x = rng.standard_normal((m, k)).astype(np.float32)
        y = mm.forward(torch.from_numpy(x).cuda(), mode=tq.Mode.INT8_ACT)
        tq.context().poll_status()
        assert y.shape == (m, n)
        check_int8(tq, qt, blocks2d, dt, n, k, x, y, rows)
    # a row's result does not depend on the batch it is in
    assert torch.equal(mm.forward(torch.from_numpy(x[:1]).cuda(), mode=tq.Mode.INT8_ACT), y[:1])


@pytest.mark.parametrize("m", [1, 8])
def test_mixed_type_qkv_launch_at_the_8b_shapes(tq, m):
    """attn_q|k (Q4_K) and attn_v (Q6_K) of Qwen3-8B in one call: 4096 / 1024 / 1024 x 4096."""
    k = 4096
    rng = np.random.default_rng(SEED + 4096 + m)
    parts = [(Q4_K, 4096), (Q4_K, 1024), (Q6_K, 1024)]
    made = [make(tq, dt, n, k, SEED + 50 + i) for i, (dt, n) in enumerate(parts)]
    mms = [tq.QMatMul.from_arc(qt) for qt, _ in made]
    x = rng.standard_normal((m, k)).astype(np.float32)
    l0 = tq.context().launch_count()
    ys = tq.QMatMul.forward_multi(mms, torch.from_numpy(x).cuda(), mode=tq.Mode.INT8_ACT)
    launches = tq.context().launch_count() - l0
    assert launches <= (1 if m == 1 else 2)
    tq.context().poll_status()
    for (dt, n), (qt, b2d), y, mm in zip(parts, made, ys, mms):
        check_int8(tq, qt, b2d, dt, n, k, x, y, sample_rows(n, 128, rng))
        assert torch.equal(mm.forward(torch.from_numpy(x).cuda(), mode=tq.Mode.INT8_ACT), y)


@pytest.mark.parametrize("dt,n,k,m,nrows", [
    (Q4_K, 12288, 4096, 2048, 192),    # cfg3 ffn_gate, grid.y = 8
    (Q4_K, 12288, 4096, 8192, 96),     # grid.y = 32
    (Q6_K, 4096, 12288, 2048, 128),    # cfg3 ffn_down
    (Q6_K, 4096, 12288, 8192, 64),
    (Q5_K, 12288, 4096, 512, 192),     # cfg3 Q5_K_M variant
    (Q6_K, 5120, 25600, 64, 256),      # cfg5 ffn_down, decode batch: split-K over 40 tiles
    (Q4_K, 1024, 5120, 64, 256),       # cfg5 attn_k: 8 tiles -> 16 K splits of 5 blocks
    (Q6_K, 5120, 25600, 4096, 48),     # cfg5 prefill
    (Q8_0, 2560, 8192, 1024, 128),     # cfg4 Q8_0 ffn_down, prefill
], ids=["gate_q4k_m2048", "gate_q4k_m8192", "down_q6k_m2048", "down_q6k_m8192", "gate_q5k_m512",
        "down32b_q6k_m64_splitk", "k32b_q4k_m64_splitk", "down32b_q6k_m4096", "down3b_q8_0_m1024"])
def test_tensor_core_scheme_at_config_shapes(tq, dt, n, k, m, nrows):
    rng = np.random.default_rng(SEED + n + k + m)
    qt, blocks2d = make(tq, dt, n, k, SEED + n + 1)
    mm = tq.QMatMul.from_arc(qt)
    rows = sample_rows(n, nrows, rng)
    xb = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)   # prefill feeds bf16
    y = mm.forward(xb, mode=tq.Mode.TENSOR_CORE)
    tq.context().poll_status()
    assert y.shape == (m, n)
    w = blocks2d[torch.from_numpy(rows).cuda()].cpu().numpy()
    # all activation rows against the sampled weight rows (f64 accumulation on the host)
    want = oracle.matmul_f64(dt, w, len(rows), k, xb.float().cpu().numpy())
    got = y[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    assert oracle.rel_fro(got, want) < TOL
    worst = max(oracle.rel_fro(got[r], want[r]) for r in (0, 1, m // 2, m - 2, m - 1))
    assert worst < 2 * TOL
    assert torch.isfinite(y).all()
