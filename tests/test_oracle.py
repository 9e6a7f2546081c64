"""CPU oracle against the golden vectors produced by the independent gguf-py codec, plus
self-consistency properties of the restated quantizers and dot products."""
import os

import numpy as np
import pytest

import oracle

TYPES = [oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K]
ids = [oracle.NAMES[t] for t in TYPES]


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_dequantize_matches_gguf_golden_bit_exact(dt, golden_dir):
    g = np.load(os.path.join(golden_dir, "gguf_dequantize.npz"))
    name = oracle.NAMES[dt]
    blocks, want = g[f"{name}_blocks"], g[f"{name}_f32"]
    be = oracle.block_elems(dt)
    got = oracle.dequantize(dt, blocks.reshape(1, -1), be * blocks.shape[0]).reshape(-1, be)
    assert np.array_equal(bits(got), bits(want))


def test_q8_0_quantizer_matches_gguf_golden_bit_exact(golden_dir):
    g = np.load(os.path.join(golden_dir, "gguf_quantize_q8_0.npz"))
    got = oracle.quantize(oracle.Q8_0, g["x"])
    assert np.array_equal(got, g["blocks"])


def test_frozen_activation_blocks_and_matmuls(golden_dir):
    g = np.load(os.path.join(golden_dir, "oracle_matmul.npz"))
    x = g["act_x"]
    assert np.array_equal(oracle.quantize(oracle.Q8_K, x), g["act_q8k"])
    assert np.array_equal(oracle.quantize(oracle.Q8_0, x), g["act_q8_0"])
    k = x.shape[1]
    for dt in TYPES:
        name = oracle.NAMES[dt]
        w = g[f"{name}_w"]
        n = w.shape[0]
        y1 = oracle.qmatmul(dt, w, n, k, x, nthreads=1)
        y2 = oracle.matmul_f64(dt, w, n, k, x, nthreads=1)
        assert np.array_equal(bits(y1), bits(g[f"{name}_y_cpu_scheme"]))
        assert np.array_equal(bits(y2), bits(g[f"{name}_y_f64"]))


def test_block_geometry():
    assert [oracle.block_elems(t) for t in TYPES + [oracle.Q8_K]] == [32, 256, 256, 256, 256]
    assert [oracle.block_bytes(t) for t in TYPES + [oracle.Q8_K]] == [34, 144, 176, 210, 292]
    assert oracle.row_bytes(oracle.Q6_K, 4096) == 3360
    with pytest.raises(ValueError):
        oracle.row_bytes(oracle.Q4_K, 100)


@pytest.mark.parametrize("dt,tol", [(oracle.Q8_0, 0.01), (oracle.Q4_K, 0.10), (oracle.Q5_K, 0.05), (oracle.Q6_K, 0.03)],
                         ids=ids)
def test_weight_quantizers_round_trip_error(dt, tol):
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((32, 1024)) * 0.02).astype(np.float32)
    back = oracle.dequantize(dt, oracle.quantize(dt, w), 1024)
    assert oracle.rel_fro(back, w) < tol


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_quantizers_handle_zero_constant_and_huge_rows(dt):
    k = 512
    x = np.zeros((4, k), np.float32)
    x[1] = 3.0
    x[2] = -1e4
    x[3, ::7] = 1e-30
    back = oracle.dequantize(dt, oracle.quantize(dt, x), k)
    assert np.all(np.isfinite(back))
    assert np.array_equal(back[0], np.zeros(k, np.float32))
    assert oracle.rel_fro(back[1], x[1]) < 0.02
    assert oracle.rel_fro(back[2], x[2]) < 0.02


def test_q8k_semantics_largest_element_maps_to_minus_128_and_clamps():
    k = 256
    x = np.linspace(-1, 1, k, dtype=np.float32)
    x[5] = -4.0
    b = oracle.quantize(oracle.Q8_K, x[None])[0]
    assert b[:4].view(np.float32)[0] == np.float32(1 / 32)
    qs = b[4:260].view(np.int8)
    assert qs[5] == -128
    assert np.array_equal(b[260:].view(np.int16), qs.reshape(16, 16).astype(np.int32).sum(1).astype(np.int16))
    x[5], x[9] = 4.0, -4.0           # first of two equal magnitudes wins; its mirror clamps at 127
    b = oracle.quantize(oracle.Q8_K, x[None])[0]
    assert b[:4].view(np.float32)[0] == np.float32(-1 / 32)
    qs = b[4:260].view(np.int8)
    assert qs[5] == -128 and qs[9] == 127
    assert np.array_equal(oracle.quantize(oracle.Q8_K, np.zeros((1, k), np.float32))[0], np.zeros(292, np.uint8))


@pytest.mark.parametrize("dt", TYPES, ids=ids)
def test_cpu_scheme_close_to_f64_oracle_and_row_independent(dt):
    rng = np.random.default_rng(11)
    n, k = 40, 768
    w = oracle.quantize(dt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    x = rng.standard_normal((6, k)).astype(np.float32)
    y_int = oracle.qmatmul(dt, w, n, k, x)
    y_f64 = oracle.matmul_f64(dt, w, n, k, x)
    assert oracle.rel_fro(y_int, y_f64) < 2e-2      # activation rounding noise, ~5-8e-3
    # each output row depends on its own activation row only
    y_one = oracle.qmatmul(dt, w, n, k, x[3:4])
    assert np.array_equal(bits(y_one[0]), bits(y_int[3]))
    # thread count does not change results
    assert np.array_equal(bits(oracle.qmatmul(dt, w, n, k, x, nthreads=1)), bits(y_int))


def test_f16_conversions_exhaustive():
    lib = oracle._load()
    hs = np.arange(0, 65536, 7, dtype=np.uint32)
    want = hs.astype(np.uint16).view(np.float16).astype(np.float32)
    got = np.array([lib.tqo_f16_to_f32(int(h)) for h in hs], dtype=np.float32)
    ok = ~np.isnan(want)
    assert np.array_equal(bits(got[ok]), bits(want[ok]))
    rng = np.random.default_rng(3)
    t = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32)
    with np.errstate(over="ignore"):
        ref = t.astype(np.float16).view(np.uint16)
    mine = np.array([lib.tqo_f32_to_f16(float(v)) for v in t], dtype=np.uint16)
    assert np.array_equal(ref, mine)


def _tie_rows():
    """Rows whose scaled values are exact .5 ties: block maximum +-1.0 -> |iscale| = 128 (or 127)."""
    k = 256
    j = np.arange(k - 1)
    x = np.empty((2, k), np.float32)
    x[0, :-1] = ((2 * j + 1) % 255) / np.float32(256.0) * np.where(j % 3 == 0, -1, 1)
    x[0, -1] = 1.0
    x[1, :-1] = ((2 * j + 1) % 253) / np.float32(254.0) * np.where(j % 2 == 0, -1, 1)   # ties for divisor 127
    x[1, -1] = -1.0
    return x


def _q(blocks):
    return blocks.reshape(-1, 292)[:, 4:260].view(np.int8).astype(np.int32), blocks.reshape(-1, 292)[:, :4].view(np.float32)


def test_q8k_default_is_candles_published_quantizer_ties_away_from_zero():
    assert oracle.q8k_variant() == 0x180          # divisor 128, negative-scale convention, ties away
    x = _tie_rows()[:1]
    q, d = _q(oracle.quantize(oracle.Q8_K, x))
    v = np.float32(-128.0) * x[0]
    want = np.where(v >= 0, np.floor(v + 0.5), -np.floor(-v + 0.5)).astype(np.int32)   # half away from zero
    assert np.array_equal(q[0], np.minimum(want, 127))
    assert q[0, -1] == -128 and d[0, 0] == np.float32(-1 / 128)
    assert np.count_nonzero(np.abs(v - np.trunc(v)) == 0.5) > 100      # half of the row is exact ties


@pytest.mark.parametrize("defs,check", [
    ({"TQO_Q8K_ROUND_HALF_EVEN": 1}, "even"),
    ({"TQO_Q8K_DIVISOR": 127}, "div127"),
    ({"TQO_Q8K_NEG_SCALE": 0}, "pos"),
    ({"TQO_Q8K_DIVISOR": 127, "TQO_Q8K_NEG_SCALE": 0, "TQO_Q8K_ROUND_HALF_EVEN": 1}, "ggml127"),
], ids=["ties_to_even", "divisor_127", "positive_scale", "all_three"])
def test_q8k_switches_each_change_exactly_their_choice(defs, check):
    x = _tie_rows()
    base_q, base_d = _q(oracle.quantize(oracle.Q8_K, x))
    q, d = _q(oracle.quantize_q8k_variant(x, **defs))
    if check == "even":
        v = np.float32(-128.0) * x[0]
        assert np.array_equal(q[0], np.minimum(np.rint(v).astype(np.int32), 127))     # numpy rint: ties to even
        assert not np.array_equal(q[0], base_q[0]) and np.array_equal(d, base_d)
    elif check == "div127":
        assert d[0, 0] == np.float32(1.0) / (np.float32(-127.0) / np.float32(1.0)) and q[0, -1] == -127
        assert d[1, 0] == np.float32(1.0) / (np.float32(-127.0) / np.float32(-1.0)) and q[1, -1] == -127
    elif check == "pos":
        assert np.all(d > 0) and q[0, -1] == 127 and q[1, -1] == -128      # +1.0 * 128 clamps, -1.0 * 128 fits
        assert np.array_equal(q[1], base_q[1])                             # row 1's maximum is negative: same scale
    else:
        v = (np.float32(127.0) / np.float32(1.0)) * x[1]
        assert np.array_equal(q[1], np.rint(v).astype(np.int32)) and d[1, 0] == np.float32(1.0) / np.float32(127.0)
    # group sums always match the quants
    b = oracle.quantize_q8k_variant(x, **defs).reshape(-1, 292)
    assert np.array_equal(b[:, 260:].view(np.int16), q.reshape(2, 16, 16).sum(2).astype(np.int16))
