"""CUDA path against the CPU oracle, through the C ABI (tur_b200.quantized is a thin ctypes
layer). Bit-exact for dequantize and activation blocks; matmul within 2e-3 relative
Frobenius error of the oracle of the same scheme (the north-star tolerance)."""
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TYPES = [oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K]
ids = [oracle.NAMES[t] for t in TYPES]
TOL = 2e-3
SEED = 299792458


@pytest.fixture(scope="module")
def tq():
    import tur_b200
    from tur_b200 import quantized
    assert torch.cuda.is_available()
    return quantized


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def make_weight(dt, n, k, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    return oracle.quantize(dt, w)


# ---------------------------------------------------------------- dequantize

@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_dequantize_golden_blocks_bit_exact(tq, dt, golden_dir):
    g = np.load(os.path.join(golden_dir, "gguf_dequantize.npz"))
    name = oracle.NAMES[dt]
    blocks, want = g[f"{name}_blocks"], g[f"{name}_f32"]
    nb, be = blocks.shape[0], oracle.block_elems(dt)
    # lay the blocks out as a [rows, cols] tensor in several shapes (1 row, ragged rows)
    for rows in (1, 3, nb):
        if nb % rows:
            continue
        cols = nb // rows * be
        qt = tq.QTensor.new(blocks, tq.GgmlDType(dt), (rows, cols))
        got = qt.dequantize().cpu().numpy()
        assert np.array_equal(bits(got), bits(want.reshape(rows, cols)))


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("n,k", [(1, 256), (17, 2560), (33, 4096), (130, 512)])
def test_dequantize_matches_oracle_bit_exact(tq, dt, n, k):
    w = make_weight(dt, n, k, SEED + n + k)
    qt = tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))
    assert qt.shape() == (n, k) and qt.dtype() == tq.GgmlDType(dt) and qt.storage_size_in_bytes() == w.size
    want = oracle.dequantize(dt, w, k)
    got = qt.dequantize().cpu().numpy()
    assert np.array_equal(bits(got), bits(want))
    # from device-resident wire blocks too
    qt2 = tq.QTensor.new(torch.from_numpy(w).cuda(), tq.GgmlDType(dt), (n, k))
    assert np.array_equal(bits(qt2.dequantize().cpu().numpy()), bits(want))
    # half outputs are the exact f32 rounded once
    h = qt.dequantize(torch.float16).cpu()
    assert torch.equal(h, torch.from_numpy(want).to(torch.float16))
    b = qt.dequantize(torch.bfloat16).cpu()
    assert torch.equal(b, torch.from_numpy(want).to(torch.bfloat16))


# ---------------------------------------------------------------- activation quantization

def test_activation_blocks_golden_bit_exact(tq, golden_dir):
    g = np.load(os.path.join(golden_dir, "oracle_matmul.npz"))
    x = torch.from_numpy(g["act_x"]).cuda()
    assert np.array_equal(tq.quantize_act(x, tq.GgmlDType.Q8K).cpu().numpy(), g["act_q8k"])
    assert np.array_equal(tq.quantize_act(x, tq.GgmlDType.Q8_0).cpu().numpy(), g["act_q8_0"])
    g2 = np.load(os.path.join(golden_dir, "gguf_quantize_q8_0.npz"))
    got = tq.quantize_act(torch.from_numpy(g2["x"]).cuda(), tq.GgmlDType.Q8_0).cpu().numpy()
    assert np.array_equal(got, g2["blocks"])


@pytest.mark.parametrize("m,k", [(1, 256), (5, 4096), (16, 12288), (64, 2560)])
def test_activation_blocks_match_oracle_bit_exact(tq, m, k):
    rng = np.random.default_rng(SEED + 10**6 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0, :256] = 0.0
    if m > 1:
        x[1] *= 1e-3
        x[1, 3], x[1, 77] = 2.5, -2.5      # equal magnitudes: first wins, mirror clamps
    xd = torch.from_numpy(x).cuda()
    for fmt, ofmt in ((tq.GgmlDType.Q8K, oracle.Q8_K), (tq.GgmlDType.Q8_0, oracle.Q8_0)):
        assert np.array_equal(tq.quantize_act(xd, fmt).cpu().numpy(), oracle.quantize(ofmt, x))
    xb = xd.to(torch.bfloat16)
    want = oracle.quantize(oracle.Q8_K, xb.float().cpu().numpy())
    assert np.array_equal(tq.quantize_act(xb, tq.GgmlDType.Q8K).cpu().numpy(), want)


# ---------------------------------------------------------------- matmul

@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_matmul_golden(tq, dt, golden_dir):
    g = np.load(os.path.join(golden_dir, "oracle_matmul.npz"))
    name = oracle.NAMES[dt]
    w, x = g[f"{name}_w"], g["act_x"]
    n, k = w.shape[0], x.shape[1]
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    xd = torch.from_numpy(x).cuda()
    y_int = mm.forward(xd, mode=tq.Mode.INT8_ACT).cpu().numpy()
    y_f32 = mm.forward(xd, mode=tq.Mode.EXACT_F32).cpu().numpy()
    assert oracle.rel_fro(y_int, g[f"{name}_y_cpu_scheme"]) < 1e-5
    assert oracle.rel_fro(y_f32, g[f"{name}_y_f64"]) < 1e-5


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("n,k,m", [(16, 256, 1), (3, 512, 2), (1024, 4096, 1), (1024, 4096, 4), (100, 2560, 8),
                                   (640, 2560, 16), (257, 1024, 5), (4096, 12288, 1), (2048, 1024, 33),
                                   # activation planes copied into shared memory (3 < M <= 16), odd plane sizes
                                   (300, 4096, 12), (64, 256, 9), (512, 12288, 4), (40, 768, 13), (96, 8192, 7),
                                   # several row-tiles per CTA
                                   (9600, 512, 1), (9500, 256, 5), (10000, 1024, 16), (9700, 2560, 3)])
def test_matmul_matches_oracle_of_same_scheme(tq, dt, n, k, m):
    w = make_weight(dt, n, k, SEED + 1000 + n)
    rng = np.random.default_rng(SEED + 10**6 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    xd = torch.from_numpy(x).cuda()
    y_int = mm.forward(xd, mode=tq.Mode.INT8_ACT).cpu().numpy()
    want_int = oracle.qmatmul(dt, w, n, k, x)
    assert y_int.shape == (m, n)
    assert oracle.rel_fro(y_int, want_int) < TOL
    assert oracle.rel_fro(y_int, want_int) < 1e-5      # only the f32 summation order differs
    if n * k * m <= 4096 * 4096 * 4:
        y_f32 = mm.forward(xd, mode=tq.Mode.EXACT_F32).cpu().numpy()
        want_f64 = oracle.matmul_f64(dt, w, n, k, x)
        assert oracle.rel_fro(y_f32, want_f64) < TOL
        assert oracle.rel_fro(y_f32, want_f64) < 1e-5
        # the two schemes differ by the activation rounding noise only
        assert oracle.rel_fro(y_int, want_f64) < 2e-2


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("n,k,m", [(4096, 2560, 1), (1024, 5120, 3), (2560, 6400, 16), (272, 1280, 1)])
def test_streaming_pipeline_is_race_free_when_stages_are_partly_filled(tq, dt, n, k, m):
    """In-features that do not fill the 8-tile stages evenly (10, 20, 25, 5 tiles per row) leave
    consumer warps without a tile in some stages; repeated launches must stay bit-identical and
    correct, and no kernel may give up a wait."""
    w = make_weight(dt, n, k, SEED + 4000 + k)
    rng = np.random.default_rng(SEED + 5)
    x = rng.standard_normal((m, k)).astype(np.float32)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    xd = torch.from_numpy(x).cuda()
    first = mm.forward(xd, mode=tq.Mode.INT8_ACT)
    for _ in range(40):
        assert torch.equal(mm.forward(xd, mode=tq.Mode.INT8_ACT), first)
    tq.context().poll_status()
    assert oracle.rel_fro(first.cpu().numpy(), oracle.qmatmul(dt, w, n, k, x)) < 1e-5


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_rows_are_independent_of_batch_size_and_bias_is_added(tq, dt):
    """tur's tests rely on a token's result not depending on its batch neighbours
    (tests/pipeline_integration.rs:275-369, tests/engine_integration.rs:171-251)."""
    n, k = 512, 2048
    w = make_weight(dt, n, k, SEED + 5)
    rng = np.random.default_rng(SEED + 6)
    x = torch.from_numpy(rng.standard_normal((16, k)).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    for mode in (tq.Mode.INT8_ACT, tq.Mode.EXACT_F32):
        y16 = mm.forward(x, mode=mode)
        for rows in (slice(0, 1), slice(3, 5), slice(7, 16)):
            assert torch.equal(mm.forward(x[rows], mode=mode), y16[rows])
        yb = mm.forward(x, bias=bias, mode=mode)
        assert torch.equal(yb, y16 + bias)
    # rank-3 input keeps its leading dims (src/models/qwen3.rs:269-274 feeds [B, L, hidden])
    y3 = mm.forward(x.reshape(2, 8, k), mode=tq.Mode.INT8_ACT)
    assert y3.shape == (2, 8, n) and torch.equal(y3.reshape(16, n), mm.forward(x, mode=tq.Mode.INT8_ACT))


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_bf16_activations(tq, dt):
    n, k, m = 256, 1024, 4
    w = make_weight(dt, n, k, SEED + 9)
    rng = np.random.default_rng(SEED + 10)
    xb = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    xr = xb.float().cpu().numpy()
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    assert oracle.rel_fro(mm.forward(xb, mode=tq.Mode.INT8_ACT).cpu().numpy(), oracle.qmatmul(dt, w, n, k, xr)) < 1e-5
    assert oracle.rel_fro(mm.forward(xb, mode=tq.Mode.EXACT_F32).cpu().numpy(), oracle.matmul_f64(dt, w, n, k, xr)) < 1e-5


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_host_buffer_entry(tq, dt):
    n, k, m = 300, 1024, 3
    w = make_weight(dt, n, k, SEED + 11)
    rng = np.random.default_rng(SEED + 12)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    y = mm.forward(torch.from_numpy(x), bias=torch.from_numpy(bias)).numpy()
    want = oracle.qmatmul(dt, w, n, k, x) + bias
    assert oracle.rel_fro(y, want) < 1e-5


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_shards_reassemble_the_unsharded_result(tq, dt):
    """Column-parallel shards (row slices) are bit-exact pieces; row-parallel shards (column
    slices) sum to the full result up to f32 reassociation."""
    n, k, m = 96, 2048, 4
    w = make_weight(dt, n, k, SEED + 13)
    rng = np.random.default_rng(SEED + 14)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
    qt = tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))
    full = tq.QMatMul(qt).forward(x, mode=tq.Mode.INT8_ACT)
    parts = [tq.QMatMul(qt.slice_rows(r0, cnt)).forward(x, mode=tq.Mode.INT8_ACT) for r0, cnt in ((0, 32), (32, 48), (80, 16))]
    assert torch.equal(torch.cat(parts, dim=1), full)
    acc = torch.zeros_like(full)
    for c0, cnt in ((0, 768), (768, 256), (1024, 1024)):
        acc += tq.QMatMul(qt.slice_cols(c0, cnt)).forward(x[:, c0:c0 + cnt].contiguous(), mode=tq.Mode.INT8_ACT)
    assert oracle.rel_fro(acc.cpu().numpy(), full.cpu().numpy()) < 1e-5
    assert np.array_equal(bits(qt.slice_cols(768, 256).dequantize().cpu().numpy()),
                          bits(oracle.dequantize(dt, w, k)[:, 768:1024]))


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("n,k,m", [(128, 256, 256), (200, 512, 77), (304, 1024, 48), (1024, 2048, 64), (1024, 4096, 512), (4096, 1024, 300), (272, 2560, 1024)])
def test_tensor_core_mode_matches_f64_oracle(tq, dt, n, k, m):
    """tcgen05 f16 path: within 2e-3 relative Frobenius error of dequantize-then-matmul."""
    w = make_weight(dt, n, k, SEED + 2000 + n)
    rng = np.random.default_rng(SEED + 10**6 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0] *= 3.0e5                     # a row that would overflow f16 without the row scaling
    if m > 2:
        x[2] = 0.0
    bias = rng.standard_normal(n).astype(np.float32)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    xd = torch.from_numpy(x).cuda()
    y = mm.forward(xd, bias=torch.from_numpy(bias).cuda(), mode=tq.Mode.TENSOR_CORE).cpu().numpy()
    tq.context().poll_status()
    want = oracle.matmul_f64(dt, w, n, k, x) + bias
    assert y.shape == (m, n)
    for rows in (slice(0, 1), slice(1, m)):      # the huge row must not hide errors elsewhere
        assert oracle.rel_fro(y[rows], want[rows]) < TOL
    # bf16 activations (the prefill configs feed bf16): exact in f16 for N(0,1) values
    xb = torch.from_numpy(x[1:]).cuda().to(torch.bfloat16)
    yb = mm.forward(xb, mode=tq.Mode.TENSOR_CORE).cpu().numpy()
    assert oracle.rel_fro(yb, oracle.matmul_f64(dt, w, n, k, xb.float().cpu().numpy())) < TOL
    # AUTO picks this path for prefill-sized M and results do not depend on the batch
    if 17 < m <= 64:
        # decode batches: split-K depends on the weight's shape only, not on the batch
        y17 = mm.forward(xd[:17], mode=tq.Mode.TENSOR_CORE)
        assert torch.equal(y17, mm.forward(xd, mode=tq.Mode.TENSOR_CORE)[:17])
    if m > 64:
        assert torch.equal(mm.forward(xd, mode=tq.Mode.AUTO), mm.forward(xd, mode=tq.Mode.TENSOR_CORE))
        y2 = mm.forward(xd[: m // 2 + 1], mode=tq.Mode.TENSOR_CORE)
        assert torch.equal(y2, mm.forward(xd, mode=tq.Mode.TENSOR_CORE)[: m // 2 + 1])


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("m", [1, 5, 16])
def test_one_launch_for_linears_sharing_x(tq, dt, m):
    """q|k|v / gate|up style call: same results as separate calls (f32 summation order aside),
    ragged row counts, per-part bias."""
    k = 1024
    shapes = [272, 64, 1000]
    rng = np.random.default_rng(SEED + 77 + m)
    ws = [make_weight(dt, n, k, SEED + 300 + n) for n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))) for w, n in zip(ws, shapes)]
    x = rng.standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    bias1 = torch.from_numpy(rng.standard_normal(shapes[1]).astype(np.float32)).cuda()
    l0 = tq.context().launch_count()
    ys = tq.QMatMul.forward_multi(mms, xd, biases=[None, bias1, None], mode=tq.Mode.INT8_ACT)
    assert tq.context().launch_count() - l0 <= 2   # one GEMV kernel (+ a quantization launch beyond a few rows)
    tq.context().poll_status()
    for i, (w, n) in enumerate(zip(ws, shapes)):
        want = oracle.qmatmul(dt, w, n, k, x) + (bias1.cpu().numpy() if i == 1 else 0)
        assert ys[i].shape == (m, n)
        assert oracle.rel_fro(ys[i].cpu().numpy(), want) < 1e-5
    # other type combinations go out as one launch per type (or a mixed launch) and still agree
    other = TYPES[(TYPES.index(dt) + 1) % len(TYPES)]
    w2 = make_weight(other, 48, k, SEED + 9)
    mixed = [mms[0], tq.QMatMul.from_arc(tq.QTensor.new(w2, tq.GgmlDType(other), (48, k)))]
    y2 = tq.QMatMul.forward_multi(mixed, xd, mode=tq.Mode.INT8_ACT)
    assert oracle.rel_fro(y2[1].cpu().numpy(), oracle.qmatmul(other, w2, 48, k, x)) < 1e-5
    assert oracle.rel_fro(y2[0].cpu().numpy(), oracle.qmatmul(dt, ws[0], shapes[0], k, x)) < 1e-5


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("m", [1, 6])
def test_joint_launch_gives_the_same_bits_as_separate_launches(tq, dt, m):
    """Which CTA computes a row-tile must not show in the result: a joint launch over two
    weights (another split of the row-tiles over CTAs) equals the two separate launches bit for
    bit, and repeated launches repeat exactly."""
    k = 512
    shapes = [6000, 4100]
    rng = np.random.default_rng(SEED + 99 + m)
    ws = [make_weight(dt, n, k, SEED + 500 + n) for n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))) for w, n in zip(ws, shapes)]
    xd = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
    joint = [y.clone() for y in tq.QMatMul.forward_multi(mms, xd, mode=tq.Mode.INT8_ACT)]
    for _ in range(3):
        again = tq.QMatMul.forward_multi(mms, xd, mode=tq.Mode.INT8_ACT)
        assert all(torch.equal(a, b) for a, b in zip(again, joint))
    tq.context().poll_status()
    for mm, y in zip(mms, joint):
        assert torch.equal(mm.forward(xd, mode=tq.Mode.INT8_ACT), y)
    want = oracle.qmatmul(dt, ws[1], shapes[1], k, xd.cpu().numpy())
    assert oracle.rel_fro(joint[1].cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("dt", [oracle.Q4_K, oracle.Q5_K], ids=lambda d: oracle.NAMES[d])
@pytest.mark.parametrize("m", [1, 3, 8, 12])
def test_mixed_type_launch_for_attn_qkv(tq, dt, m):
    """The K-quant mixes keep attn_v in Q6_K beside Q4_K / Q5_K attn_q and attn_k: one call, and
    up to 8 rows one kernel launch, with the bits of the separate launches."""
    k = 1024
    shapes = [(dt, 272), (dt, 64), (oracle.Q6_K, 1000)]
    rng = np.random.default_rng(SEED + 123 + m)
    ws = [make_weight(t, n, k, SEED + 700 + n) for t, n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(t), (n, k))) for w, (t, n) in zip(ws, shapes)]
    x = rng.standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    bias2 = torch.from_numpy(rng.standard_normal(1000).astype(np.float32)).cuda()
    l0 = tq.context().launch_count()
    ys = tq.QMatMul.forward_multi(mms, xd, biases=[None, None, bias2], mode=tq.Mode.INT8_ACT)
    launches = tq.context().launch_count() - l0
    if m == 1:
        assert launches == 1
    tq.context().poll_status()
    for i, (mm, (t, n)) in enumerate(zip(mms, shapes)):
        sep = mm.forward(xd, bias=bias2 if i == 2 else None, mode=tq.Mode.INT8_ACT)
        assert torch.equal(ys[i], sep)
        want = oracle.qmatmul(t, ws[i], n, k, x) + (bias2.cpu().numpy() if i == 2 else 0)
        assert oracle.rel_fro(ys[i].cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_embedding_lookup_equals_dequantize_then_index(tq, dt):
    """tur dequantizes token_embd and indexes the f32 table (src/models/layers/mod.rs:30-48);
    the lookup on the quantized table must give those bits, for any id order and repeats."""
    n, k = 1000, 2560
    w = make_weight(dt, n, k, SEED + 31)
    qt = tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))
    full = qt.dequantize()
    rng = np.random.default_rng(SEED + 32)
    ids = torch.from_numpy(rng.integers(0, n, size=(3, 37))).cuda()
    ids[0, 0], ids[0, 1], ids[2, 36] = 0, n - 1, 15
    got = qt.embedding(ids)
    assert got.shape == (3, 37, k)
    assert torch.equal(got, full[ids])
    assert torch.equal(qt.embedding(ids, torch.bfloat16), full[ids].to(torch.bfloat16))
    assert np.array_equal(got[0, 1].cpu().numpy(), oracle.dequantize(dt, w, k)[n - 1])
    assert qt.embedding(ids[:0]).shape == (0, 37, k)
    tq.context().poll_status()
    # an id outside the table: zero row, reported at the next status poll, context stays usable
    bad = torch.tensor([5, n, 7], device="cuda")
    out = qt.embedding(bad)
    assert torch.equal(out[0], full[5]) and torch.equal(out[2], full[7]) and not out[1].any()
    with pytest.raises(tq.TurqError) as e:
        tq.context().poll_status()
    assert e.value.status == 1
    tq.context().poll_status()
    assert torch.equal(qt.embedding(ids), full[ids])


@pytest.mark.parametrize("second", [oracle.Q4_K, oracle.Q6_K], ids=["same_type", "mixed_types"])
@pytest.mark.parametrize("m", [1, 5])
def test_joint_launch_with_row_tiles_cut_between_ctas(tq, second, m):
    """601 row-tiles of 16 K-tiles on 296 CTA slots: whole row-tiles per CTA would idle a third of
    the slots, so the tiles are dealt out evenly and row-tiles are cut between CTAs (partial sums
    handed over) - here across two weights of one launch, of one type or of two."""
    k = 4096
    shapes = [(oracle.Q4_K, 5000), (second, 4600)]
    rng = np.random.default_rng(SEED + 555 + m)
    ws = [make_weight(t, n, k, SEED + 900 + n) for t, n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(t), (n, k))) for w, (t, n) in zip(ws, shapes)]
    x = rng.standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    first = [y.clone() for y in tq.QMatMul.forward_multi(mms, xd, mode=tq.Mode.INT8_ACT)]
    for _ in range(3):
        again = tq.QMatMul.forward_multi(mms, xd, mode=tq.Mode.INT8_ACT)
        assert all(torch.equal(a, b) for a, b in zip(again, first))
    tq.context().poll_status()
    for y, w, (t, n) in zip(first, ws, shapes):
        assert oracle.rel_fro(y.cpu().numpy(), oracle.qmatmul(t, w, n, k, x)) < 1e-5


@pytest.mark.parametrize("dt", [oracle.Q4_K, oracle.Q5_K, oracle.Q6_K], ids=["Q4_K", "Q5_K", "Q6_K"])
@pytest.mark.parametrize("n,k", [(272, 2560), (5000, 4096), (1040, 12288)], ids=["partly_filled_stages", "cut_row_tiles", "staged_planes"])
def test_single_row_tile_function_gives_the_bits_of_a_batch_row(tq, dt, n, k):
    """One activation row takes a tile function of its own in the K-quant GEMV (sub-blocks in the
    MMA's columns instead of activation rows). Its sums must be the general function's: row 0 of
    a 2-, 5- and 11-row batch, through whole and cut row-tiles and both activation routes."""
    w = make_weight(dt, n, k, SEED + 77 + n)
    rng = np.random.default_rng(SEED + 78 + k)
    x = rng.standard_normal((11, k)).astype(np.float32)
    x[0, ::7] *= 40.0   # wide range inside the blocks of the row under test
    xd = torch.from_numpy(x).cuda()
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    y1 = mm.forward(xd[:1], mode=tq.Mode.INT8_ACT)
    for rows in (2, 5, 11):
        assert torch.equal(mm.forward(xd[:rows], mode=tq.Mode.INT8_ACT)[:1], y1)
    assert oracle.rel_fro(y1.cpu().numpy(), oracle.qmatmul(dt, w, n, k, x[:1])) < 1e-5
    tq.context().poll_status()


def test_single_row_tile_function_in_a_mixed_type_launch(tq):
    """attn_q|k|v of the K-quant mixes as one launch at one row (both single-row tile functions in
    one kernel) against the same launch at three rows."""
    k = 4096
    shapes = [(oracle.Q4_K, 4096), (oracle.Q4_K, 1024), (oracle.Q6_K, 1024)]
    ws = [make_weight(t, n, k, SEED + 1200 + i) for i, (t, n) in enumerate(shapes)]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(t), (n, k))) for w, (t, n) in zip(ws, shapes)]
    x = np.random.default_rng(SEED + 1210).standard_normal((3, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    one = [y.clone() for y in tq.QMatMul.forward_multi(mms, xd[:1], mode=tq.Mode.INT8_ACT)]
    three = tq.QMatMul.forward_multi(mms, xd, mode=tq.Mode.INT8_ACT)
    for a, b, w, (t, n) in zip(one, three, ws, shapes):
        assert torch.equal(a, b[:1])
        assert oracle.rel_fro(a.cpu().numpy(), oracle.qmatmul(t, w, n, k, x[:1])) < 1e-5
    tq.context().poll_status()


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_weight_quantizer_writes_the_oracle_quantizer_bytes(tq, dt):
    """QTensor::quantize (candle-core; the benchmark configurations quantize their synthetic
    weights with it). The device quantizer must write the bytes of the CPU restatement: seeded
    N(0, 0.02) rows as the configurations prescribe, plus blocks that take the search's side
    exits (all zero, constant, all positive, all negative, one outlier, tiny and huge ranges)."""
    from tur_b200.quantized import quantize_weights
    n, k = 37, 2048
    rng = np.random.default_rng(SEED + 4242 + dt)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[0, :256] = 0.0
    w[1, :256] = 0.75
    w[2, :256] = np.abs(w[2, :256]) + 0.01
    w[3, :256] = -np.abs(w[3, :256]) - 0.01
    w[4, 17] = 9.0
    w[5, :256] *= 1e-20
    w[6, :256] *= 1e20
    w[7, 32:64] = 0.0          # one empty sub-block inside a live block
    w[8, :256] = np.round(w[8, :256] * 400) / 400   # many rounding ties
    want = oracle.quantize(dt, w)
    got = quantize_weights(torch.from_numpy(w).cuda(), tq.GgmlDType(dt))
    tq.context().poll_status()
    got = got.cpu().numpy().reshape(-1)
    want = np.asarray(want).view(np.uint8).reshape(-1)
    assert got.size == want.size
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, f"{bad.size} bytes differ, first at {bad[:8]} (block bytes {oracle.block_bytes(dt)})"
    # and the tensor made from them is the oracle's tensor
    qt = tq.QTensor.quantize(torch.from_numpy(w).cuda(), tq.GgmlDType(dt))
    assert qt.shape() == (n, k) and qt.dtype() == tq.GgmlDType(dt)
    # (the huge-range row overflows the f16 block scale: inf and inf * 0 on both sides)
    assert np.array_equal(qt.dequantize().cpu().numpy(), oracle.dequantize(dt, want, k), equal_nan=True)


def test_weight_quantizer_rejects_what_it_cannot_do(tq):
    from tur_b200.quantized import quantize_weights
    x = torch.zeros(4, 256, device="cuda")
    with pytest.raises(tq.TurqError) as e:
        quantize_weights(x, tq.GgmlDType.Q8K)           # an activation format, not a weight type
    assert e.value.status == 3
    with pytest.raises(tq.TurqError) as e:
        quantize_weights(x[:, :100].contiguous(), tq.GgmlDType.Q4K)   # not whole blocks
    assert e.value.status == 2
    with pytest.raises(tq.TurqError):
        quantize_weights(x.cpu(), tq.GgmlDType.Q4K)     # no CPU fallback
    tq.context().poll_status()


@pytest.mark.parametrize("dt,n,k,m", [(oracle.Q8_0, 256, 1728, 100), (oracle.Q4_K, 256, 1792, 40), (oracle.Q6_K, 384, 1792, 40),
                                      (oracle.Q5_K, 128, 1792, 17)],
                         ids=["q8_0_27_blocks_unsplit", "q4k_split_9_9_10", "q6k_split_9_9_10", "q5k_split"])
def test_tensor_core_k_loop_with_an_odd_number_of_blocks(tq, dt, n, k, m):
    """The GEMM's MMA thread handles two 64-wide K-blocks per barrier round; a K loop (or a CTA's
    share of it under split-K) with an odd count ends on a half-filled pair."""
    w = make_weight(dt, n, k, SEED + 3100 + k)
    rng = np.random.default_rng(SEED + 3101 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    y = mm.forward(xb, mode=tq.Mode.TENSOR_CORE)
    assert torch.equal(y, mm.forward(xb, mode=tq.Mode.TENSOR_CORE))
    assert oracle.rel_fro(y.cpu().numpy(), oracle.matmul_f64(dt, w, n, k, xb.float().cpu().numpy())) < 2e-3
    tq.context().poll_status()


def test_no_kernel_gave_up_a_wait(tq):
    tq.context().poll_status()


def test_error_paths_return_status_not_crash(tq):
    w = make_weight(oracle.Q4_K, 16, 256, 1)
    with pytest.raises(tq.TurqError) as e:
        tq.QTensor.new(w, tq.GgmlDType.Q4K, (16, 512))          # byte count mismatch
    assert e.value.status == 2
    with pytest.raises(tq.TurqError) as e:
        tq.QTensor.new(w, tq.GgmlDType.Q4K, (16, 100))          # not whole blocks
    assert e.value.status == 2
    with pytest.raises(tq.TurqError) as e:
        tq.QTensor.new(w, tq.GgmlDType.F32, (16, 256))          # not a quantized weight type
    assert e.value.status == 3
    qt = tq.QTensor.new(w, tq.GgmlDType.Q4K, (16, 256))
    with pytest.raises(tq.TurqError):
        tq.QMatMul(qt).forward(torch.zeros(2, 128, device="cuda"))
    with pytest.raises(tq.TurqError) as e:
        qt.slice_rows(8, 8)
    assert e.value.status == 2
    with pytest.raises(tq.TurqError) as e:
        qt.slice_cols(0, 100)
    assert e.value.status == 2


def test_q8k_ties_round_as_the_oracle_does_and_the_build_switches_agree(tq):
    """Exact .5 ties after scaling (common for bf16 and low-mantissa inputs): the library and the
    oracle must have been built with the same Q8_K switches and then agree bit for bit."""
    from tur_b200 import _lib
    assert _lib.load().turq_q8k_variant() == oracle.q8k_variant()
    k = 512
    j = np.arange(255)
    x = np.zeros((4, k), np.float32)
    x[0, :255] = ((2 * j + 1) % 255) / np.float32(256.0) * np.where(j % 3 == 0, -1, 1)
    x[0, 255] = 1.0
    x[1, :255] = -x[0, :255]
    x[1, 255] = -1.0
    x[2, 256:511] = (j + 0.5) / np.float32(128.0) * np.where(j % 2 == 0, -1, 1)
    x[2, 511] = -2.0
    x[3] = np.round(np.random.default_rng(SEED).standard_normal(k) * 8) / 16     # low-mantissa values
    xd = torch.from_numpy(x).cuda()
    assert np.array_equal(tq.quantize_act(xd, tq.GgmlDType.Q8K).cpu().numpy(), oracle.quantize(oracle.Q8_K, x))
    xb = xd.to(torch.bfloat16)
    assert np.array_equal(tq.quantize_act(xb, tq.GgmlDType.Q8K).cpu().numpy(),
                          oracle.quantize(oracle.Q8_K, xb.float().cpu().numpy()))
    # the GEMV's own quantization (in-kernel for one row, staged planes for more) follows suit
    for dt in (oracle.Q4_K, oracle.Q6_K):
        w = make_weight(dt, 64, k, SEED + 41)
        mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (64, k)))
        for rows in (slice(0, 1), slice(0, 4)):
            y = mm.forward(xd[rows], mode=tq.Mode.INT8_ACT).cpu().numpy()
            assert oracle.rel_fro(y, oracle.qmatmul(dt, w, 64, k, x[rows])) < 1e-6


def test_operands_are_validated_before_any_launch(tq):
    """A tensor on another device, of another element type or with strides would make a kernel
    read memory it must not: the host layer refuses it with a status instead."""
    w = make_weight(oracle.Q4_K, 32, 256, 3)
    mm = tq.QMatMul(tq.QTensor.new(w, tq.GgmlDType.Q4K, (32, 256)))
    x = torch.zeros(2, 256, device="cuda")
    with pytest.raises(tq.TurqError) as e:
        mm.forward(x, bias=torch.zeros(32, device="cuda", dtype=torch.float16))
    assert e.value.status == 3
    with pytest.raises(tq.TurqError) as e:
        mm.forward(x, bias=torch.zeros(32))                                   # bias on the host
    assert e.value.status == 1
    with pytest.raises(tq.TurqError) as e:
        mm.forward(x, bias=torch.zeros(31, device="cuda"))
    assert e.value.status == 2
    with pytest.raises(tq.TurqError) as e:
        mm.forward(x, out=torch.zeros(2, 64, device="cuda")[:, ::2])          # strided output
    assert e.value.status == 1
    with pytest.raises(tq.TurqError) as e:
        mm.forward(x, out=torch.zeros(2, 32, device="cuda", dtype=torch.bfloat16))
    assert e.value.status == 3
    with pytest.raises(tq.TurqError) as e:
        mm.forward(x, out=torch.zeros(2, 32))                                 # output on the host
    assert e.value.status == 1
    with pytest.raises(tq.TurqError) as e:
        tq.QMatMul.forward_multi([mm, mm], x, outs=[torch.zeros(2, 32, device="cuda"), torch.zeros(2, 16, device="cuda")])
    assert e.value.status == 2
    with pytest.raises(tq.TurqError) as e:
        mm.forward(torch.zeros(2, 256), out=torch.zeros(2, 32, device="cuda"))  # host x, device out
    assert e.value.status == 1
    assert torch.equal(mm.forward(x), torch.zeros(2, 32, device="cuda"))      # and the context still works


@pytest.mark.parametrize("dt", TYPES, ids=ids)
@pytest.mark.parametrize("pinned", [True, False], ids=["page_locked", "pageable"])
def test_host_entries_for_several_weights_in_one_round_trip(tq, dt, pinned):
    """turq_qmatmul_multi_host: q|k|v or gate|up from one host x. Page-locked buffers take the
    copy-free route (x read and y written in place by the kernels), pageable ones are copied;
    both must give the bits of the device-tensor call."""
    k, shapes, m = 1024, [272, 64, 1000], 3
    rng = np.random.default_rng(SEED + 321)
    ws = [make_weight(dt, n, k, SEED + 800 + n) for n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))) for w, n in zip(ws, shapes)]
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
    if pinned:
        x = x.pin_memory()
    want = tq.QMatMul.forward_multi(mms, x.cuda(), mode=tq.Mode.INT8_ACT)
    got = tq.QMatMul.forward_multi(mms, x, mode=tq.Mode.INT8_ACT)
    for g, wnt, w, n in zip(got, want, ws, shapes):
        assert not g.is_cuda and g.shape == (m, n)
        assert torch.equal(g, wnt.cpu())
        assert oracle.rel_fro(g.numpy(), oracle.qmatmul(dt, w, n, k, x.numpy())) < 1e-5
    # with a bias (copied route) and through the single-weight entry
    bias = torch.from_numpy(rng.standard_normal(shapes[1]).astype(np.float32))
    got_b = tq.QMatMul.forward_multi(mms, x, biases=[None, bias, None], mode=tq.Mode.INT8_ACT)
    assert torch.equal(got_b[1], want[1].cpu() + bias) and torch.equal(got_b[0], want[0].cpu())
    assert torch.equal(mms[2].forward(x, mode=tq.Mode.INT8_ACT), want[2].cpu())
    # repeated calls reuse the same buffers
    for _ in range(3):
        again = tq.QMatMul.forward_multi(mms, x, mode=tq.Mode.INT8_ACT)
        assert all(torch.equal(a, b) for a, b in zip(again, got))
    # other schemes go through the copied route and still agree with the device call
    y_tc = mms[0].forward(x.repeat(8, 1), mode=tq.Mode.TENSOR_CORE)
    assert torch.equal(y_tc, mms[0].forward(x.repeat(8, 1).cuda(), mode=tq.Mode.TENSOR_CORE).cpu())


def test_auto_policy_pins_one_scheme_for_every_row_count_and_reserve_presizes(tq):
    """tur requires a token's result not to depend on its batch or chunk
    (tests/pipeline_integration.rs:275-369). AUTO switches scheme between 16 and 17 rows by
    default; a context with a pinned policy does not."""
    n, k = 256, 1024
    w = make_weight(oracle.Q4_K, n, k, SEED + 61)
    ctx = tq.new_context()
    ctx.reserve(64, k, n)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType.Q4K, (n, k), ctx=ctx))
    x = torch.from_numpy(np.random.default_rng(SEED + 62).standard_normal((40, k)).astype(np.float32)).cuda()
    y_auto = mm.forward(x, mode=tq.Mode.AUTO)
    assert torch.equal(y_auto, mm.forward(x, mode=tq.Mode.TENSOR_CORE))
    assert not torch.equal(y_auto[:8], mm.forward(x[:8], mode=tq.Mode.AUTO))        # default: scheme depends on M
    for policy in (tq.Mode.INT8_ACT, tq.Mode.TENSOR_CORE, tq.Mode.EXACT_F32):
        ctx.set_auto_policy(policy)
        y40 = mm.forward(x, mode=tq.Mode.AUTO)
        assert torch.equal(y40, mm.forward(x, mode=policy))
        for rows in (slice(0, 1), slice(5, 13), slice(0, 17)):
            assert torch.equal(mm.forward(x[rows], mode=tq.Mode.AUTO), y40[rows])
    ctx.set_auto_policy(tq.Mode.AUTO)
    assert torch.equal(mm.forward(x, mode=tq.Mode.AUTO), y_auto)
    with pytest.raises(tq.TurqError):
        ctx.reserve(0, k, n)
    ctx.poll_status()


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_tensor_core_mode_keeps_its_accuracy_for_tiny_and_huge_rows(tq, dt):
    """Rows of 1e-6 magnitude would sink into f16 subnormals and rows of 1e+6 overflow without
    the per-row power-of-two scaling in front of the f16 conversion."""
    n, k, m = 256, 1024, 96
    w = make_weight(dt, n, k, SEED + 71)
    rng = np.random.default_rng(SEED + 72)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[::3] *= np.float32(1e-6)
    x[1::3] *= np.float32(1e6)
    x[5] *= np.float32(1e-30)
    mm = tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k)))
    y = mm.forward(torch.from_numpy(x).cuda(), mode=tq.Mode.TENSOR_CORE).cpu().numpy()
    want = oracle.matmul_f64(dt, w, n, k, x)
    for r in range(m):
        assert oracle.rel_fro(y[r], want[r]) < TOL, r


def test_tensor_core_multi_call_converts_x_once_and_matches_separate_calls(tq):
    """q|k|v / gate|up in the tensor-core scheme: one f16 conversion of x for all the weights, the
    bits of the separate calls."""
    k, m = 1024, 200
    shapes = [(oracle.Q4_K, 384), (oracle.Q4_K, 128), (oracle.Q6_K, 256)]
    ws = [make_weight(t, n, k, SEED + 600 + n) for t, n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(t), (n, k))) for w, (t, n) in zip(ws, shapes)]
    x = torch.from_numpy(np.random.default_rng(SEED + 601).standard_normal((m, k)).astype(np.float32)).cuda()
    bias = torch.from_numpy(np.random.default_rng(SEED + 602).standard_normal(128).astype(np.float32)).cuda()
    sep = [mm.forward(x, bias=bias if i == 1 else None, mode=tq.Mode.TENSOR_CORE) for i, mm in enumerate(mms)]
    l0 = tq.context().launch_count()
    got = tq.QMatMul.forward_multi(mms, x, biases=[None, bias, None], mode=tq.Mode.TENSOR_CORE)
    assert tq.context().launch_count() - l0 == 1 + len(mms)          # one conversion, one GEMM per weight
    tq.context().poll_status()
    for g, s_, w, (t, n) in zip(got, sep, ws, shapes):
        assert torch.equal(g, s_)
    assert oracle.rel_fro(got[2].cpu().numpy(), oracle.matmul_f64(oracle.Q6_K, ws[2], 256, k, x.cpu().numpy())) < TOL


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_bound_host_call_reruns_on_rewritten_buffers(tq, dt):
    """turq_host_call_*: a decoder binds q|k|v (or one linear) to its page-locked buffers once and
    reruns the call after rewriting x in place; every run gives the bits of the device call."""
    k, shapes = 1024, [272, 64, 1000]
    rng = np.random.default_rng(SEED + 909)
    ws = [make_weight(dt, n, k, SEED + 900 + n) for n in shapes]
    mms = [tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))) for w, n in zip(ws, shapes)]
    for m in (1, 5, 16):
        x = torch.empty((m, k), dtype=torch.float32).pin_memory()
        call = tq.HostCall(mms, x)
        single = tq.HostCall(mms[2:], x)
        for step in range(3):
            x.copy_(torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)))     # the next token's activations
            outs = call.run()
            want = tq.QMatMul.forward_multi(mms, x.cuda(), mode=tq.Mode.INT8_ACT)
            for o, w_ in zip(outs, want):
                assert torch.equal(o, w_.cpu())
            assert torch.equal(single.run()[0], want[2].cpu())
        assert oracle.rel_fro(outs[0].numpy(), oracle.qmatmul(dt, ws[0], shapes[0], k, x.numpy())) < 1e-5
        call.close()
        single.close()
    with pytest.raises(tq.TurqError) as e:
        tq.HostCall(mms, torch.zeros((2, k)))                  # pageable memory: not bindable
    assert e.value.status == 1
    tq.context().poll_status()


def test_contexts_are_reentrant_across_threads_and_streams(tq):
    """tur runs one worker thread per model (src/server/worker.rs:63-72). Calls through different
    contexts - each with its own scratch and hand-over workspace - may run concurrently from
    different threads on different streams and must not disturb each other."""
    import threading
    n, k = 9600, 1024                                  # 600 row-tiles: split with hand-over between CTAs
    ws = {dt: make_weight(dt, n, k, SEED + 1200 + dt) for dt in (oracle.Q4_K, oracle.Q6_K)}
    xs = {m: torch.from_numpy(np.random.default_rng(SEED + m).standard_normal((m, k)).astype(np.float32)).cuda() for m in (1, 5, 12)}
    ref_mm = {dt: tq.QMatMul.from_arc(tq.QTensor.new(w, tq.GgmlDType(dt), (n, k))) for dt, w in ws.items()}
    want = {(dt, m): ref_mm[dt].forward(x, mode=tq.Mode.INT8_ACT).clone() for dt in ws for m, x in xs.items()}
    torch.cuda.synchronize()
    errors = []

    def worker(dt):
        try:
            ctx = tq.new_context()
            mm = tq.QMatMul.from_arc(tq.QTensor.new(ws[dt], tq.GgmlDType(dt), (n, k), ctx=ctx))
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for it in range(30):
                    for m, x in xs.items():
                        y = mm.forward(x, mode=tq.Mode.INT8_ACT)
                        if it % 10 == 9:
                            stream.synchronize()
                            if not torch.equal(y, want[(dt, m)]):
                                errors.append((dt, m, it))
                ctx.poll_status()
        except Exception as e:  # reported to the main thread
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(dt,)) for dt in ws for _ in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
