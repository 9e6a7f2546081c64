"""numpy/ctypes front-end of the CPU oracle (TEST INFRASTRUCTURE, not product code).

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module.
The shared library is compiled on first use with the host's own instruction set (the file
name carries a hash of the CPU flags, so a library built on one machine is never loaded on
another).

The arithmetic restates candle-core 0.10.2's CPU path behind tur's
`QTensor::dequantize` (src/weights/mod.rs:150,161) and `QMatMul::forward`
(src/models/layers/linear.rs:24); see turq_oracle.c for the pinning status.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess

import numpy as np

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, Q8_K, BF16 = 0, 1, 8, 12, 13, 14, 15, 30
NAMES = {F32: "F32", F16: "F16", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K",
         Q8_K: "Q8_K", BF16: "BF16"}
WEIGHT_TYPES = (Q8_0, Q4_K, Q5_K, Q6_K)

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def _cpu_tag() -> str:
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


def lib_path() -> str:
    return os.path.join(_HERE, f"libturq_oracle.{_cpu_tag()}.so")


def build(force: bool = False, defines: dict | None = None) -> str:
    """Compile turq_oracle.c for this host; returns the path of the shared library.
    `defines` (e.g. {"TQO_Q8K_DIVISOR": 127}) builds a variant of the Q8_K activation quantizer
    into a file of its own, named after the switches."""
    out = lib_path()
    dflags = []
    if defines:
        tag = "_".join(f"{k}{v}" for k, v in sorted(defines.items()))
        out = out[:-3] + "." + tag + ".so"
        dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    src = os.path.join(_HERE, "turq_oracle.c")
    hdr = os.path.join(_HERE, "turq_oracle.h")
    stale = (not os.path.exists(out)
             or os.path.getmtime(out) < max(os.path.getmtime(src), os.path.getmtime(hdr)))
    if force or stale:
        # several ranks may get here at once: each compiles into a file of its own and moves it
        # into place atomically, so nobody ever loads a half-written library
        tmp = f"{out}.{os.getpid()}.tmp"
        cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-ffp-contract=off",
               "-fno-fast-math", "-std=c11", *dflags, "-shared", "-o", tmp, src, "-lm"]
        try:
            subprocess.run(cmd, check=True, cwd=_HERE)
            os.replace(tmp, out)
        finally:
            if os.path.exists(tmp):
                os.remove(tmp)
    return out


def _bind(path: str):
    lib = ctypes.CDLL(path)
    i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
    lib.tqo_block_elems.argtypes = [ci]
    lib.tqo_block_bytes.argtypes = [ci]
    lib.tqo_row_bytes.argtypes = [ci, i64]
    lib.tqo_row_bytes.restype = ctypes.c_size_t
    lib.tqo_dequantize.argtypes = [ci, vp, vp, i64, i64]
    lib.tqo_quantize.argtypes = [ci, vp, vp, i64, i64]
    lib.tqo_qmatmul.argtypes = [ci, vp, i64, i64, vp, i64, vp, ci]
    lib.tqo_matmul_f64.argtypes = [ci, vp, i64, i64, vp, i64, vp, ci]
    lib.tqo_vec_dot.argtypes = [ci, vp, vp, i64]
    lib.tqo_vec_dot.restype = ctypes.c_float
    lib.tqo_f32_to_f16.argtypes = [ctypes.c_float]
    lib.tqo_f32_to_f16.restype = ctypes.c_uint16
    lib.tqo_f16_to_f32.argtypes = [ctypes.c_uint16]
    lib.tqo_f16_to_f32.restype = ctypes.c_float
    lib.tqo_num_threads.restype = ci
    lib.tqo_q8k_variant.restype = ci
    return lib


def _load():
    global _lib
    if _lib is None:
        _lib = _bind(build())
    return _lib


def q8k_variant() -> int:
    """Q8_K quantizer switches this oracle was built with: divisor | 0x100 (negative-scale
    convention) | 0x200 (ties to even). The CUDA library reports the same word."""
    return _load().tqo_q8k_variant()


def quantize_q8k_variant(x: np.ndarray, **defines) -> np.ndarray:
    """Q8_K blocks of x [nrows, k] from an oracle built with other TQO_Q8K_* switches."""
    lib = _bind(build(defines=defines))
    x = np.ascontiguousarray(x, dtype=np.float32)
    nrows, k = x.shape
    out = np.empty((nrows, (k // 256) * 292), dtype=np.uint8)
    if lib.tqo_quantize(Q8_K, _ptr(x), _ptr(out), nrows, k) != 0:
        raise ValueError("tqo_quantize failed")
    return out


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def block_elems(dtype: int) -> int:
    return _load().tqo_block_elems(dtype)


def block_bytes(dtype: int) -> int:
    return _load().tqo_block_bytes(dtype)


def row_bytes(dtype: int, k: int) -> int:
    rb = _load().tqo_row_bytes(dtype, k)
    if rb == 0 and k != 0:
        raise ValueError(f"k={k} is not a multiple of the {NAMES.get(dtype, dtype)} block size")
    return rb


def num_threads() -> int:
    return _load().tqo_num_threads()


def quantize(dtype: int, x: np.ndarray) -> np.ndarray:
    """f32 [nrows, k] -> uint8 [nrows, row_bytes]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    nrows, k = x.shape
    out = np.empty((nrows, row_bytes(dtype, k)), dtype=np.uint8)
    if _load().tqo_quantize(dtype, _ptr(x), _ptr(out), nrows, k) != 0:
        raise ValueError("tqo_quantize failed")
    return out


def dequantize(dtype: int, blocks: np.ndarray, k: int) -> np.ndarray:
    """uint8 [nrows, row_bytes] -> f32 [nrows, k]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rb = row_bytes(dtype, k)
    nrows = blocks.size // rb if rb else 0
    assert blocks.size == nrows * rb, "byte count is not a whole number of rows"
    out = np.empty((nrows, k), dtype=np.float32)
    if _load().tqo_dequantize(dtype, _ptr(blocks), _ptr(out), nrows, k) != 0:
        raise ValueError("tqo_dequantize failed")
    return out


def act_type(dtype: int) -> int:
    """Activation block format the CPU scheme pairs with a weight type."""
    return Q8_0 if dtype == Q8_0 else Q8_K


def qmatmul(dtype: int, w: np.ndarray, n: int, k: int, x: np.ndarray, nthreads: int = 0) -> np.ndarray:
    """CPU quantized scheme: y[m, n] = quantize_act(x)[m] . W[n]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    assert w.size == n * row_bytes(dtype, k)
    y = np.empty((x.shape[0], n), dtype=np.float32)
    if _load().tqo_qmatmul(dtype, _ptr(w), n, k, _ptr(x), x.shape[0], _ptr(y), nthreads) != 0:
        raise ValueError("tqo_qmatmul failed")
    return y


def matmul_f64(dtype: int, w: np.ndarray, n: int, k: int, x: np.ndarray, nthreads: int = 0) -> np.ndarray:
    """Dequantize-then-matmul with f64 accumulation, returned as f32."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    assert w.size == n * row_bytes(dtype, k)
    y = np.empty((x.shape[0], n), dtype=np.float32)
    if _load().tqo_matmul_f64(dtype, _ptr(w), n, k, _ptr(x), x.shape[0], _ptr(y), nthreads) != 0:
        raise ValueError("tqo_matmul_f64 failed")
    return y


def rel_fro(a: np.ndarray, b: np.ndarray) -> float:
    """Relative Frobenius error ||a - b|| / ||b|| in f64."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))
