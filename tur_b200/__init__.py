"""tur_b200: B200 (sm_100a) kernels for tur's quantized-linear path behind a C ABI.

`tur_b200.quantized` mirrors the candle names tur uses on this path (GgmlDType, QTensor,
QMatMul) and `tur_b200.linear` mirrors tur's own LinearX (src/models/layers/linear.rs)."""
from .quantized import GgmlDType, QMatMul, QTensor, TurqError, Mode, context, new_context, topk, HostCall  # noqa: F401
from .linear import LinearX, linear  # noqa: F401
