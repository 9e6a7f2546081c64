"""Fused neighbours of the linears against numpy restatements on top of the CPU oracle:
SwiGLU over ffn_gate|up (src/models/qwen3.rs:160-166), RMSNorm feeding the projections
(qwen3.rs:633-638) and the head's top-k (src/backend/engine.rs:528-529, 810-824)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
SEED = 299792458
TYPES = [oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K]
ids = [oracle.NAMES[t] for t in TYPES]


@pytest.fixture(scope="module")
def tq():
    from tur_b200 import quantized
    assert torch.cuda.is_available()
    return quantized


def make_weight(dt, n, k, seed):
    rng = np.random.default_rng(seed)
    return oracle.quantize(dt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))


def silu(v):
    v = v.astype(np.float32)
    return v / (np.float32(1) + np.exp(-v, dtype=np.float32))


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("n,k,m", [(12288, 1024, 1), (4800, 512, 5), (9600, 256, 12), (320, 2048, 3), (8192, 2560, 33)])
def test_swiglu_over_gate_and_up(tq, dt, n, k, m):
    """Big shapes take the single interleaved launch, small ones (few row-tiles) the two-step
    route; both equal silu(gate) * up of the separate products."""
    wg, wu = make_weight(dt, n, k, SEED + n), make_weight(dt, n, k, SEED + n + 1)
    gate = tq.QMatMul.from_arc(tq.QTensor.new(wg, tq.GgmlDType(dt), (n, k)))
    up = tq.QMatMul.from_arc(tq.QTensor.new(wu, tq.GgmlDType(dt), (n, k)))
    x = np.random.default_rng(SEED + m).standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    l0 = tq.context().launch_count()
    got = tq.QMatMul.swiglu(gate, up, xd, mode=tq.Mode.INT8_ACT)
    launches = tq.context().launch_count() - l0
    tq.context().poll_status()
    g = gate.forward(xd, mode=tq.Mode.INT8_ACT)
    u = up.forward(xd, mode=tq.Mode.INT8_ACT)
    want_dev = (g / (1 + torch.exp(-g))) * u
    assert got.shape == (m, n)
    assert oracle.rel_fro(got.cpu().numpy(), want_dev.cpu().numpy()) < 1e-6
    want = silu(oracle.qmatmul(dt, wg, n, k, x)) * oracle.qmatmul(dt, wu, n, k, x)
    assert oracle.rel_fro(got.cpu().numpy(), want) < 1e-5
    if n >= 4800 and m <= 8:
        assert launches <= 2          # one GEMV (+ a quantization launch for wide or multi-row inputs)
    # rows stay independent of the batch
    assert torch.equal(tq.QMatMul.swiglu(gate, up, xd[:1], mode=tq.Mode.INT8_ACT), got[:1])
    # the tensor-core scheme goes the two-step route
    if m == 33:
        got_tc = tq.QMatMul.swiglu(gate, up, xd, mode=tq.Mode.TENSOR_CORE).cpu().numpy()
        want_tc = silu(oracle.matmul_f64(dt, wg, n, k, x)) * oracle.matmul_f64(dt, wu, n, k, x)
        assert oracle.rel_fro(got_tc, want_tc) < 4e-3


def rmsnorm_ref(x, w, eps):
    x = x.astype(np.float32)
    ms = (x.astype(np.float64) ** 2).mean(axis=1, keepdims=True)
    denom = np.sqrt(ms + eps).astype(np.float32)
    return (x / denom) * w.astype(np.float32)


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("k,m", [(1024, 1), (4096, 1), (2560, 6), (4096, 16)])
def test_rmsnorm_feeding_the_projections(tq, dt, k, m):
    shapes = [272, 64, 1000]
    rng = np.random.default_rng(SEED + k + m)
    ws = [make_weight(dt, n, k, SEED + 40 + n) for n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))) for w, n in zip(ws, shapes)]
    x = (rng.standard_normal((m, k)) * 3.0).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    eps = 1e-6
    xd, nwd = torch.from_numpy(x).cuda(), torch.from_numpy(nw).cuda()
    outs, h = tq.QMatMul.rmsnorm_forward_multi(mms, xd, nwd, eps, mode=tq.Mode.INT8_ACT, return_normed=True)
    tq.context().poll_status()
    h_ref = rmsnorm_ref(x, nw, eps)
    assert np.max(np.abs(h.cpu().numpy() - h_ref) / (np.abs(h_ref) + 1e-6)) < 1e-5
    # the linears consumed exactly the h that was written out
    for o, mm in zip(outs, mms):
        assert torch.equal(o, mm.forward(h, mode=tq.Mode.INT8_ACT))
    for o, w, n in zip(outs, ws, shapes):
        assert oracle.rel_fro(o.cpu().numpy(), oracle.qmatmul(dt, w, n, k, h.cpu().numpy())) < 1e-5
        assert oracle.rel_fro(o.cpu().numpy(), oracle.qmatmul(dt, w, n, k, h_ref)) < 2e-3
    # without writing h, and with a bias; bf16 input
    bias = torch.from_numpy(rng.standard_normal(shapes[1]).astype(np.float32)).cuda()
    outs2 = tq.QMatMul.rmsnorm_forward_multi(mms, xd, nwd, eps, biases=[None, bias, None], mode=tq.Mode.INT8_ACT)
    assert torch.equal(outs2[0], outs[0]) and torch.equal(outs2[1], outs[1] + bias)
    xb = xd.to(torch.bfloat16)
    outs3 = tq.QMatMul.rmsnorm_forward_multi(mms, xb, nwd, eps, mode=tq.Mode.INT8_ACT)
    h3 = rmsnorm_ref(xb.float().cpu().numpy(), nw, eps)
    assert oracle.rel_fro(outs3[2].cpu().numpy(), oracle.qmatmul(dt, ws[2], shapes[2], k, h3)) < 2e-3
    # other schemes read the normalised rows
    o_f32 = tq.QMatMul.rmsnorm_forward_multi(mms[:1], xd, nwd, eps, mode=tq.Mode.EXACT_F32)[0]
    assert oracle.rel_fro(o_f32.cpu().numpy(), oracle.matmul_f64(dt, ws[0], shapes[0], k, h_ref)) < 1e-4


@pytest.mark.parametrize("n,m,k", [(151936, 2, 1), (151936, 3, 64), (5000, 4, 8), (100, 1, 64), (2048, 1, 5), (2049, 2, 3)])
def test_topk_matches_a_stable_sort(tq, n, m, k):
    rng = np.random.default_rng(SEED + n + k)
    v = rng.standard_normal((m, n)).astype(np.float32)
    v[0, ::7] = np.float32(0.5)                   # many ties: lower id must win
    v[0, n // 2] = np.float32(9.0)
    if n > 10:
        v[-1, 3], v[-1, 9] = np.float32(7.0), np.float32(7.0)
        v[-1, 5] = np.nan                         # ranks lowest
    vd = torch.from_numpy(v).cuda()
    got_v, got_i = tq.topk(vd, k, id_offset=1000)
    vv = np.where(np.isnan(v), -np.inf, v)
    order = np.lexsort((np.arange(n)[None, :].repeat(m, 0), -vv), axis=1)[:, :k]     # value desc, id asc
    kk = min(k, n)
    assert np.array_equal(got_i.cpu().numpy()[:, :kk], order[:, :kk] + 1000)
    assert np.array_equal(got_v.cpu().numpy()[:, :kk], np.take_along_axis(vv, order[:, :kk], 1))
    if k > n:
        assert np.all(got_i.cpu().numpy()[:, n:] == np.iinfo(np.int32).max) and np.all(np.isneginf(got_v.cpu().numpy()[:, n:]))


def test_lm_head_topk_and_sharded_merge(tq):
    """Greedy / top-k straight from the head, and a vocabulary-sharded head: each shard's k best
    with id offsets, merged, equal the unsharded k best."""
    n, kdim, m, k = 20480, 1024, 3, 16
    w = make_weight(oracle.Q6_K, n, kdim, SEED + 77)
    qt = tq.QTensor.new(w, tq.GgmlDType.Q6K, (n, kdim))
    mm = tq.QMatMul.from_arc(qt)
    x = torch.from_numpy(np.random.default_rng(SEED + 78).standard_normal((m, kdim)).astype(np.float32)).cuda()
    logits = torch.empty((m, n), device="cuda")
    vals, idx = mm.lm_head_topk(x, k, mode=tq.Mode.INT8_ACT, logits_out=logits)
    tq.context().poll_status()
    assert torch.equal(logits, mm.forward(x, mode=tq.Mode.INT8_ACT))
    sv, si = torch.sort(logits, dim=1, descending=True, stable=True)
    assert torch.equal(vals, sv[:, :k]) and torch.equal(idx.long(), si[:, :k])
    g_vals, g_idx = mm.lm_head_topk(x, 1, mode=tq.Mode.INT8_ACT)          # greedy, logits kept internal
    assert torch.equal(g_idx[:, 0].long(), logits.argmax(dim=1)) and torch.equal(g_vals[:, 0], logits.max(dim=1).values)
    # four vocabulary shards
    cand_v, cand_i = [], []
    for r in range(4):
        sh = tq.QMatMul.from_arc(qt.slice_rows(r * 5120, 5120))
        v_r, i_r = sh.lm_head_topk(x, k, id_offset=r * 5120, mode=tq.Mode.INT8_ACT)
        cand_v.append(v_r)
        cand_i.append(i_r)
    mv, mi = tq.topk(torch.cat(cand_v, 1).contiguous(), k, ids=torch.cat(cand_i, 1).contiguous())
    assert torch.equal(mv, vals) and torch.equal(mi, idx)
