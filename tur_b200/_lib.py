"""ctypes binding of libturq.so: one Python function per symbol declared in include/turq.h.

The library is the product; this file adds no arithmetic. Loading fails loudly when the
shared object is missing (there is no CPU or PyTorch fallback)."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TURQ_LIBRARY_PATH points at another build of the same library (e.g. one compiled with
# -DTURQ_TUNING or other Q8_K switches); default: the in-tree build
LIB_PATH = os.environ.get("TURQ_LIBRARY_PATH") or os.path.join(_HERE, "libturq.so")

c_i32, c_i64, c_sz, c_vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t, ctypes.c_void_p
PP = ctypes.POINTER(c_vp)

# name -> (restype, argtypes); kept in step with include/turq.h (a test checks it)
SIGNATURES = {
    "turq_version": (c_i32, []),
    "turq_q8k_variant": (c_i32, []),
    "turq_status_string": (ctypes.c_char_p, [c_i32]),
    "turq_block_elems": (c_i32, [c_i32]),
    "turq_block_bytes": (c_i32, [c_i32]),
    "turq_row_bytes": (c_sz, [c_i32, c_i64]),
    "turq_ctx_create": (c_i32, [c_i32, PP]),
    "turq_ctx_destroy": (c_i32, [c_vp]),
    "turq_last_error": (ctypes.c_char_p, [c_vp]),
    "turq_ctx_launch_count": (c_i64, [c_vp]),
    "turq_ctx_poll_status": (c_i32, [c_vp, c_vp]),
    "turq_ctx_reserve": (c_i32, [c_vp, c_i64, c_i64, c_i64]),
    "turq_ctx_set_auto_policy": (c_i32, [c_vp, c_i32]),
    "turq_qtensor_from_host": (c_i32, [c_vp, c_i32, c_i64, c_i64, c_vp, c_sz, PP]),
    "turq_qtensor_from_device": (c_i32, [c_vp, c_i32, c_i64, c_i64, c_vp, c_sz, c_vp, PP]),
    "turq_qtensor_slice_rows": (c_i32, [c_vp, c_vp, c_i64, c_i64, PP]),
    "turq_qtensor_slice_cols": (c_i32, [c_vp, c_vp, c_i64, c_i64, PP]),
    "turq_qtensor_free": (c_i32, [c_vp]),
    "turq_qtensor_info": (c_i32, [c_vp, ctypes.POINTER(c_i32), ctypes.POINTER(c_i64),
                                  ctypes.POINTER(c_i64), ctypes.POINTER(c_sz)]),
    "turq_dequantize": (c_i32, [c_vp, c_vp, c_i32, c_vp, c_vp]),
    "turq_embedding": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i32, c_vp, c_vp]),
    "turq_quantize_act": (c_i32, [c_vp, c_i32, c_vp, c_i32, c_i64, c_i64, c_vp, c_vp]),
    "turq_quantize_weights": (c_i32, [c_vp, c_i32, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "turq_qmatmul": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_i32, c_vp, c_vp]),
    "turq_qmatmul_multi": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_i32, c_i64, c_vp, c_i32, c_vp, c_vp]),
    "turq_qmatmul_host": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_vp, c_i32, c_vp]),
    "turq_qmatmul_multi_host": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_i64, c_vp, c_i32, c_vp]),
    "turq_host_call_create": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_i64, c_vp, PP]),
    "turq_host_call_run": (c_i32, [c_vp]),
    "turq_host_call_destroy": (c_i32, [c_vp]),
    "turq_qmatmul_static": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp, c_vp]),
    "turq_qmatmul_swiglu": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_i32, c_vp]),
    "turq_rmsnorm_qmatmul_multi": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_i32, c_i64, c_vp, ctypes.c_float, c_vp, c_vp, c_i32, c_vp, c_vp]),
    "turq_topk": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i32, c_i32, c_vp, c_vp, c_vp]),
    "turq_lm_head_topk": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_i32, c_i32, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "turq_tp_create": (c_i32, [c_vp, c_i32, c_i32, c_sz, PP]),
    "turq_tp_export": (c_i32, [c_vp, c_vp]),
    "turq_tp_connect": (c_i32, [c_vp, c_vp]),
    "turq_tp_destroy": (c_i32, [c_vp]),
    "turq_tp_set_wait_limit": (c_i32, [c_vp, c_i64]),
    "turq_tp_set_fuse_limit": (c_i32, [c_vp, c_i64]),
    "turq_tp_set_twoshot_limit": (c_i32, [c_vp, c_i64]),
    "turq_tp_set_chunk_rows": (c_i32, [c_vp, c_i64]),
    "turq_tp_reset": (c_i32, [c_vp]),
    "turq_tp_allreduce": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_vp]),
    "turq_tp_allgather": (c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "turq_qmatmul_rowparallel": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_i32, c_vp, c_vp]),
    "turq_qmatmul_gather": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp, c_i32, c_vp, c_vp]),
    "turq_tp_connect_loopback": (c_i32, [c_vp]),
    "turq_tp_loopback_fill": (c_i32, [c_vp, c_i32, c_vp, c_i64, c_i32, c_vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Returns the loaded library, raising if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tur_b200.build` (needs nvcc). "
            "This package has no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is absent
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
