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
