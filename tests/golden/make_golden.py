"""Generates tests/golden/*.npz. Run from the repository root: python tests/golden/make_golden.py

Two families of vectors:
  * `gguf_*`  - expected values come from the independent numpy codec of the `gguf` python
                package (version recorded in the file): dequantize of Q8_0/Q4_K/Q5_K/Q6_K
                blocks and the Q8_0 quantizer. They pin the CPU oracle.
  * `oracle_*` - expected values come from the CPU oracle itself (Q8_K activation blocks,
                 both matmul oracles). They freeze the oracle's behaviour and give the CUDA
                 tests inputs that do not depend on a quantizer run.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
import oracle  # noqa: E402

SEED = 299792458  # the reference's default seed (src/backend/engine.rs:60)
HERE = os.path.dirname(os.path.abspath(__file__))


def scrub_f16(blocks2d: np.ndarray, col: int) -> None:
    """Make the f16 at byte column `col` finite (clear one exponent bit of inf/nan)."""
    hi = blocks2d[:, col + 1]
    bad = (hi & 0x7C) == 0x7C
    hi[bad] &= 0xBF


def f16_cols(dtype: int):
    return {oracle.Q8_0: (0,), oracle.Q4_K: (0, 2), oracle.Q5_K: (0, 2), oracle.Q6_K: (208,)}[dtype]


def special_blocks(dtype: int, rng) -> np.ndarray:
    """Hand-built edge blocks: all zero, all ones bits in the quants, largest finite and
    negative scales, extreme 6-bit sub-scales."""
    bb = oracle.block_bytes(dtype)
    out = []
    z = np.zeros(bb, np.uint8)
    out.append(z.copy())
    for scale_bits in (0x7BFF, 0xFBFF, 0x0001, 0x8001, 0x3C00, 0xBC00):  # max, -max, tiny, -tiny, 1, -1
        b = np.full(bb, 0xFF, np.uint8)
        for c in f16_cols(dtype):
            b[c] = scale_bits & 0xFF
            b[c + 1] = scale_bits >> 8
        out.append(b)
        b2 = rng.integers(0, 256, bb, dtype=np.uint8)
        for c in f16_cols(dtype):
            b2[c] = scale_bits & 0xFF
            b2[c + 1] = scale_bits >> 8
        out.append(b2)
    if dtype == oracle.Q6_K:
        b = np.zeros(bb, np.uint8)          # every q = 0 -> value -32*scale
        b[192:208] = 0x80                   # int8 scale -128
        b[208], b[209] = 0x00, 0x3C
        out.append(b)
        b = np.full(bb, 0xFF, np.uint8)     # every q = 63 -> value +31*scale
        b[192:208] = 0x7F
        b[208], b[209] = 0x00, 0x3C
        out.append(b)
    return np.stack(out)


def main() -> None:
    import gguf
    from gguf import quants
    from gguf.constants import GGMLQuantizationType as T

    gmap = {oracle.Q8_0: T.Q8_0, oracle.Q4_K: T.Q4_K, oracle.Q5_K: T.Q5_K, oracle.Q6_K: T.Q6_K}
    rng = np.random.default_rng(SEED)
    K = 512

    # ---- gguf-pinned dequantize vectors
    import importlib.metadata
    deq = {"gguf_version": np.array(importlib.metadata.version("gguf"))}
    for dt, gt in gmap.items():
        name = oracle.NAMES[dt]
        bb, be = oracle.block_bytes(dt), oracle.block_elems(dt)
        w = (rng.standard_normal((6, K)) * 0.02).astype(np.float32)
        w[1] *= 50.0
        w[2, : K // 2] = 0.0
        w[3] = np.abs(w[3])
        qb = oracle.quantize(dt, w).reshape(-1, bb)
        rnd = rng.integers(0, 256, (24, bb), dtype=np.uint8)
        for c in f16_cols(dt):
            scrub_f16(rnd, c)
        blocks = np.concatenate([qb, rnd, special_blocks(dt, rng)], axis=0)
        with np.errstate(all="ignore"):
            exp = quants.dequantize(blocks, gt).astype(np.float32)
        assert exp.shape == (blocks.shape[0], be)
        deq[f"{name}_blocks"] = blocks
        deq[f"{name}_f32"] = exp
    np.savez_compressed(os.path.join(HERE, "gguf_dequantize.npz"), **deq)

    # ---- gguf-pinned Q8_0 quantizer vectors (weights and, in the CPU scheme, activations)
    x = rng.standard_normal((8, K)).astype(np.float32)
    x[1] *= 0.02
    x[2, :32] = 0.0
    x[3, ::2] = 0.5 * np.round(x[3, ::2] * 4)      # exact .5 ties after scaling
    x[4] = np.float32(127.0) * np.sign(x[4])
    x[5, :64] = np.linspace(-63.5, 63.5, 64, dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "gguf_quantize_q8_0.npz"), x=x,
                        blocks=quants.quantize(x, T.Q8_0))

    # ---- oracle-frozen vectors: Q8_K blocks and matmul outputs
    frozen = {}
    xa = rng.standard_normal((5, K)).astype(np.float32)
    xa[1] *= 30.0
    xa[2, :256] = 0.0
    xa[3, 7] = -xa[3].max() * 2            # largest magnitude negative
    xa[4, 9] = np.abs(xa[4]).max() * 2     # largest magnitude positive -> clamps at 127
    # exact .5 ties after scaling: block maximum +1.0 gives iscale = -128 and -(2j+1)/2 products
    xa[0, :255] = ((2 * np.arange(255) + 1) % 255 + 0.0).astype(np.float32) / np.float32(256.0) * np.where(np.arange(255) % 3 == 0, -1, 1)
    xa[0, 255] = 1.0
    frozen["act_x"] = xa
    frozen["act_q8k"] = oracle.quantize(oracle.Q8_K, xa)
    frozen["act_q8_0"] = oracle.quantize(oracle.Q8_0, xa)
    N = 24
    for dt in gmap:
        name = oracle.NAMES[dt]
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        wb = oracle.quantize(dt, w)
        frozen[f"{name}_w"] = wb
        frozen[f"{name}_y_cpu_scheme"] = oracle.qmatmul(dt, wb, N, K, xa, nthreads=1)
        frozen[f"{name}_y_f64"] = oracle.matmul_f64(dt, wb, N, K, xa, nthreads=1)
    np.savez_compressed(os.path.join(HERE, "oracle_matmul.npz"), **frozen)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
