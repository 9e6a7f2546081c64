"""Host-side mirror of the candle operator surface tur uses for quantized linears.

Names and argument meaning follow `candle_core::quantized` as called by the reference:
  GgmlDType                          block_size / type_size
  QTensor::new / dequantize / shape  src/weights/gguf_varbuilder.rs:62,73,79; src/weights/mod.rs:150
  QMatMul::from_arc / forward        src/models/layers/linear.rs:24,69
Every method is a thin call into the C ABI (include/turq.h); torch is used only to own
device memory and to name the current CUDA stream. Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib


class TurqError(RuntimeError):
    """A C-ABI call returned a non-zero turq_status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"turq status {status} ({_lib.load().turq_status_string(status).decode()}): {message}")
        self.status = status


class GgmlDType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q8_0 = 8
    Q4K = 12
    Q5K = 13
    Q6K = 14
    Q8K = 15
    BF16 = 30

    def block_size(self) -> int:
        return _lib.load().turq_block_elems(int(self))

    def type_size(self) -> int:
        return _lib.load().turq_block_bytes(int(self))


class Mode(enum.IntEnum):
    AUTO = 0
    INT8_ACT = 1
    EXACT_F32 = 2
    TENSOR_CORE = 3


_TORCH_TO_GGML = {torch.float32: GgmlDType.F32, torch.float16: GgmlDType.F16, torch.bfloat16: GgmlDType.BF16}
_GGML_TO_TORCH = {v: k for k, v in _TORCH_TO_GGML.items()}


class _Context:
    """One turq_ctx per CUDA device, created on first use."""

    def __init__(self, device: int):
        lib = _lib.load()
        handle = ctypes.c_void_p()
        st = lib.turq_ctx_create(device, ctypes.byref(handle))
        if st != 0:
            raise TurqError(st, f"turq_ctx_create(device={device}) failed")
        self.handle = handle
        self.device = device

    def check(self, st: int) -> None:
        if st != 0:
            raise TurqError(st, _lib.load().turq_last_error(self.handle).decode())

    def poll_status(self) -> None:
        """Synchronizes the current stream and raises if a kernel gave up a bounded wait."""
        self.check(_lib.load().turq_ctx_poll_status(self.handle, _stream_ptr(self.device)))

    def launch_count(self) -> int:
        return int(_lib.load().turq_ctx_launch_count(self.handle))

    def reserve(self, max_m: int, max_k: int, max_n: int) -> None:
        """Sizes the context's scratch for its largest call, so that no later call allocates
        (required before capturing calls into a CUDA graph)."""
        self.check(_lib.load().turq_ctx_reserve(self.handle, max_m, max_k, max_n))

    def set_auto_policy(self, mode: "Mode") -> None:
        """Pins what Mode.AUTO means on this context to one scheme for every row count."""
        self.check(_lib.load().turq_ctx_set_auto_policy(self.handle, int(mode)))


_contexts: dict[int, _Context] = {}


def context(device: int | torch.device | None = None) -> _Context:
    if device is None:
        device = torch.cuda.current_device() if torch.cuda.is_available() else 0
    if isinstance(device, torch.device):
        device = device.index if device.index is not None else torch.cuda.current_device()
    ctx = _contexts.get(device)
    if ctx is None:
        ctx = _contexts[device] = _Context(device)
    return ctx


def new_context(device: int | torch.device | None = None) -> _Context:
    """An additional context on the device. A context owns the scratch and hand-over
    workspace of the calls made through it, so kernels that may overlap on the GPU (linears
    issued on different streams, e.g. q / k / v of one layer) must use different contexts."""
    if device is None:
        device = torch.cuda.current_device() if torch.cuda.is_available() else 0
    if isinstance(device, torch.device):
        device = device.index if device.index is not None else torch.cuda.current_device()
    return _Context(device)


def _stream_ptr(device: int) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_operand(t: torch.Tensor, what: str, device: int, dtypes: Sequence[torch.dtype]) -> None:
    """The kernels dereference raw pointers on the weight's device: refuse, before any launch,
    a tensor that lives elsewhere, has another element type or is not dense."""
    if not t.is_cuda or t.device.index != device:
        raise TurqError(1, f"{what} lives on {t.device}, the weight on cuda:{device}")
    if t.dtype not in dtypes:
        raise TurqError(3, f"{what} has dtype {t.dtype}, expected one of {[str(d) for d in dtypes]}")
    if not t.is_contiguous():
        raise TurqError(1, f"{what} must be contiguous")


class QTensor:
    """Immutable quantized weight [rows, cols] resident on one GPU."""

    def __init__(self, handle: ctypes.c_void_p, ctx: _Context):
        self._h = handle
        self._ctx = ctx
        lib = _lib.load()
        dt, r, c, nb = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_size_t()
        ctx.check(lib.turq_qtensor_info(handle, ctypes.byref(dt), ctypes.byref(r), ctypes.byref(c), ctypes.byref(nb)))
        self._dtype, self._shape, self._nbytes = GgmlDType(dt.value), (r.value, c.value), nb.value

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.load().turq_qtensor_free(h)
            except Exception:
                pass

    @classmethod
    def new(cls, blocks: np.ndarray | bytes | torch.Tensor, dtype: GgmlDType, shape: Sequence[int],
            device: int | torch.device | None = None, ctx: Optional[_Context] = None) -> "QTensor":
        """From GGUF wire-format blocks (host bytes, or a uint8 CUDA tensor). `ctx` binds the
        tensor (and the matmuls on it) to a specific context; default: the device's shared one."""
        if len(shape) != 2:
            raise TurqError(2, f"QTensor needs a 2-D shape, got {tuple(shape)}")
        rows, cols = int(shape[0]), int(shape[1])
        lib = _lib.load()
        out = ctypes.c_void_p()
        if isinstance(blocks, torch.Tensor) and blocks.is_cuda:
            ctx = ctx or context(blocks.device)
            blocks = blocks.contiguous().view(torch.uint8)
            ctx.check(lib.turq_qtensor_from_device(ctx.handle, int(dtype), rows, cols, ctypes.c_void_p(blocks.data_ptr()),
                                                   blocks.numel(), _stream_ptr(ctx.device), ctypes.byref(out)))
            torch.cuda.current_stream(ctx.device).synchronize()
            return cls(out, ctx)
        ctx = ctx or context(device)
        if isinstance(blocks, torch.Tensor):
            blocks = blocks.contiguous().view(torch.uint8).numpy()
        buf = np.frombuffer(blocks, dtype=np.uint8) if isinstance(blocks, (bytes, bytearray)) else np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        ctx.check(lib.turq_qtensor_from_host(ctx.handle, int(dtype), rows, cols, buf.ctypes.data_as(ctypes.c_void_p),
                                             buf.size, ctypes.byref(out)))
        return cls(out, ctx)

    @classmethod
    def quantize(cls, src: torch.Tensor, dtype: GgmlDType, ctx: Optional[_Context] = None) -> "QTensor":
        """candle: QTensor::quantize(&Tensor, GgmlDType). src is a 2-D f32 CUDA tensor whose
        columns are whole blocks of `dtype` (Q8_0, Q4_K, Q5_K, Q6_K)."""
        blocks = quantize_weights(src, dtype, ctx=ctx)
        return cls.new(blocks, dtype, tuple(src.shape), ctx=ctx)

    def dtype(self) -> GgmlDType:
        return self._dtype

    def shape(self) -> tuple[int, int]:
        return self._shape

    def storage_size_in_bytes(self) -> int:
        return self._nbytes

    def device(self) -> torch.device:
        return torch.device("cuda", self._ctx.device)

    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        out = torch.empty(self._shape, dtype=out_dtype, device=self.device())
        self._ctx.check(_lib.load().turq_dequantize(self._ctx.handle, self._h, int(_TORCH_TO_GGML[out_dtype]),
                                                    ctypes.c_void_p(out.data_ptr()), _stream_ptr(self._ctx.device)))
        return out

    def embedding(self, ids: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Embedding lookup on the quantized table (tur dequantizes token_embd once and indexes
        it, src/models/layers/mod.rs:30-48): ids [...] of any integer dtype -> [..., n_cols], the
        bits `dequantize()[ids]` would give. Ids outside the table give zero rows and make the
        next `poll_status()` raise."""
        dev = self.device()
        flat = ids.reshape(-1).to(device=dev, dtype=torch.int32).contiguous()
        out = torch.empty((flat.numel(), self._shape[1]), dtype=out_dtype, device=dev)
        self._ctx.check(_lib.load().turq_embedding(self._ctx.handle, self._h, ctypes.c_void_p(flat.data_ptr()), flat.numel(),
                                                   int(_TORCH_TO_GGML[out_dtype]), ctypes.c_void_p(out.data_ptr()),
                                                   _stream_ptr(self._ctx.device)))
        return out.reshape(*ids.shape, self._shape[1])

    def slice_rows(self, row0: int, n: int) -> "QTensor":
        out = ctypes.c_void_p()
        self._ctx.check(_lib.load().turq_qtensor_slice_rows(self._ctx.handle, self._h, row0, n, ctypes.byref(out)))
        return QTensor(out, self._ctx)

    def slice_cols(self, col0: int, n: int) -> "QTensor":
        out = ctypes.c_void_p()
        self._ctx.check(_lib.load().turq_qtensor_slice_cols(self._ctx.handle, self._h, col0, n, ctypes.byref(out)))
        return QTensor(out, self._ctx)


def quantize_act(x: torch.Tensor, fmt: GgmlDType) -> torch.Tensor:
    """x [m, k] (f32/bf16, CUDA) -> uint8 [m, row_bytes] of wire-format Q8_0 / Q8_K blocks."""
    if not x.is_cuda:
        raise TurqError(8, "quantize_act needs a CUDA tensor (no CPU fallback)")
    ctx = context(x.device)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    m, k = x2.shape
    lib = _lib.load()
    rb = lib.turq_row_bytes(int(fmt), k)
    out = torch.empty((m, max(rb, 1)), dtype=torch.uint8, device=x.device)
    ctx.check(lib.turq_quantize_act(ctx.handle, int(fmt), ctypes.c_void_p(x2.data_ptr()), int(_TORCH_TO_GGML[x2.dtype]),
                                    m, k, ctypes.c_void_p(out.data_ptr()), _stream_ptr(ctx.device)))
    return out


def quantize_weights(src: torch.Tensor, dtype: GgmlDType, ctx: Optional[_Context] = None) -> torch.Tensor:
    """f32 [n, k] (CUDA) -> uint8 [n, row_bytes] of wire-format blocks of a weight type."""
    if not src.is_cuda:
        raise TurqError(8, "quantize_weights needs a CUDA tensor (no CPU fallback)")
    if src.dim() != 2 or src.dtype != torch.float32:
        raise TurqError(2, f"quantize_weights needs a 2-D f32 tensor, got {tuple(src.shape)} {src.dtype}")
    ctx = ctx or context(src.device)
    x2 = src.contiguous()
    n, k = x2.shape
    lib = _lib.load()
    rb = lib.turq_row_bytes(int(dtype), k)
    out = torch.empty((n, max(rb, 1)), dtype=torch.uint8, device=src.device)
    ctx.check(lib.turq_quantize_weights(ctx.handle, int(dtype), ctypes.c_void_p(x2.data_ptr()), n, k,
                                        ctypes.c_void_p(out.data_ptr()), _stream_ptr(ctx.device)))
    return out


class QMatMul:
    """y = x . W^T for a quantized W (candle: QMatMul::from_arc + Module::forward)."""

    def __init__(self, qtensor: QTensor, mode: Mode = Mode.AUTO):
        self.qtensor = qtensor
        self.mode = mode

    @classmethod
    def from_arc(cls, qtensor: QTensor) -> "QMatMul":
        return cls(qtensor)

    from_qtensor = from_arc

    def forward(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, mode: Optional[Mode] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [..., k] -> [..., n] f32. CUDA tensors run stream-ordered on the current stream;
        CPU tensors go through the host-buffer entry (copies inside the call)."""
        qt = self.qtensor
        n, k = qt.shape()
        if x.dim() < 1 or x.shape[-1] != k:
            raise TurqError(2, f"last dim of x {tuple(x.shape)} must equal in-features {k}")
        mode = self.mode if mode is None else mode
        lead = tuple(x.shape[:-1])
        lib = _lib.load()
        ctx = qt._ctx
        if not x.is_cuda:
            # (the common case - a dense f32 matrix - skips the conversions: this entry is called
            # once per linear and its host-side cost is part of every round trip)
            x2 = x if (x.dim() == 2 and x.dtype is torch.float32 and x.is_contiguous()) else x.reshape(-1, k).to(torch.float32).contiguous()
            if out is not None and (out.is_cuda or out.dtype != torch.float32 or not out.is_contiguous()
                                    or out.numel() != x2.shape[0] * n):
                raise TurqError(1, "out must be a contiguous f32 host tensor of m x n elements when x is a host tensor")
            y = out if out is not None else torch.empty((x2.shape[0], n), dtype=torch.float32, pin_memory=x2.is_pinned())
            b = bias.to(torch.float32).contiguous() if bias is not None else None
            ctx.check(lib.turq_qmatmul_host(ctx.handle, qt._h, x2.data_ptr(), x2.shape[0], y.data_ptr(), int(mode),
                                            b.data_ptr() if b is not None else None))
            return y if y.shape == (*lead, n) else y.reshape(*lead, n)
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        x2 = x.reshape(-1, k).contiguous()
        m = x2.shape[0]
        _check_operand(x2, "x", ctx.device, (torch.float32, torch.bfloat16))
        if bias is not None:
            _check_operand(bias, "bias", ctx.device, (torch.float32,))
            if bias.numel() != n:
                raise TurqError(2, f"bias has {bias.numel()} elements, the weight {n} rows")
        if out is not None:
            _check_operand(out, "out", ctx.device, (torch.float32,))
            if out.numel() != m * n:
                raise TurqError(2, f"out has {out.numel()} elements, expected {m} x {n}")
        y = out if out is not None else torch.empty((m, n), dtype=torch.float32, device=qt.device())
        ctx.check(lib.turq_qmatmul(ctx.handle, qt._h, ctypes.c_void_p(x2.data_ptr()), int(_TORCH_TO_GGML[x2.dtype]), m,
                                   ctypes.c_void_p(y.data_ptr()), int(mode),
                                   ctypes.c_void_p(bias.data_ptr()) if bias is not None else None,
                                   _stream_ptr(ctx.device)))
        return y.reshape(*lead, n)

    __call__ = forward

    @staticmethod
    def forward_multi(mms: Sequence["QMatMul"], x: torch.Tensor, biases: Optional[Sequence[Optional[torch.Tensor]]] = None,
                      mode: Mode = Mode.AUTO, outs: Optional[Sequence[torch.Tensor]] = None) -> list[torch.Tensor]:
        """Linears that read the same x (q|k|v, gate|up) in one call: weights of one type run
        as a single kernel launch over their concatenated rows. x [..., k] is a CUDA tensor, or a
        host tensor (then the call makes one round trip for all the weights)."""
        lib = _lib.load()
        n = len(mms)
        ctx = mms[0].qtensor._ctx
        k = mms[0].qtensor.shape()[1]
        arr = ctypes.c_void_p * n
        qts = arr(*[mm.qtensor._h for mm in mms])
        lead = tuple(x.shape[:-1])
        if not x.is_cuda:
            # host tensors: one round trip for all the weights (turq_qmatmul_multi_host)
            x2 = x if (x.dim() == 2 and x.dtype is torch.float32 and x.is_contiguous()) else x.reshape(-1, k).to(torch.float32).contiguous()
            m = x2.shape[0]
            if outs is None:
                outs = [torch.empty((m, mm.qtensor.shape()[0]), dtype=torch.float32, pin_memory=x2.is_pinned()) for mm in mms]
            for o, mm in zip(outs, mms):
                if o.is_cuda or o.dtype != torch.float32 or not o.is_contiguous() or o.numel() != m * mm.qtensor.shape()[0]:
                    raise TurqError(1, "outs must be contiguous f32 host tensors of m x n elements when x is a host tensor")
            ys = arr(*[o.data_ptr() for o in outs])
            bs, keep = None, []
            if biases is not None:
                keep = [b.to(torch.float32).contiguous() if b is not None else None for b in biases]
                bs = arr(*[b.data_ptr() if b is not None else None for b in keep])
            ctx.check(lib.turq_qmatmul_multi_host(ctx.handle, n, qts, x2.data_ptr(), m, ys, int(mode), bs))
            return [o if o.shape == (*lead, o.shape[-1]) else o.reshape(*lead, o.shape[-1]) for o in outs]
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        x2 = x.reshape(-1, k).contiguous()
        m = x2.shape[0]
        _check_operand(x2, "x", ctx.device, (torch.float32, torch.bfloat16))
        if outs is None:
            outs = [torch.empty((m, mm.qtensor.shape()[0]), dtype=torch.float32, device=ctx.device) for mm in mms]
        for i, (o, mm) in enumerate(zip(outs, mms)):
            _check_operand(o, f"outs[{i}]", ctx.device, (torch.float32,))
            if o.numel() != m * mm.qtensor.shape()[0]:
                raise TurqError(2, f"outs[{i}] has {o.numel()} elements, expected {m} x {mm.qtensor.shape()[0]}")
        ys = arr(*[ctypes.c_void_p(o.data_ptr()) for o in outs])
        bs = None
        if biases is not None:
            for i, (b, mm) in enumerate(zip(biases, mms)):
                if b is not None:
                    _check_operand(b, f"biases[{i}]", ctx.device, (torch.float32,))
                    if b.numel() != mm.qtensor.shape()[0]:
                        raise TurqError(2, f"biases[{i}] has {b.numel()} elements, the weight {mm.qtensor.shape()[0]} rows")
            bs = arr(*[ctypes.c_void_p(b.data_ptr()) if b is not None else None for b in biases])
        ctx.check(lib.turq_qmatmul_multi(ctx.handle, n, qts, ctypes.c_void_p(x2.data_ptr()), int(_TORCH_TO_GGML[x2.dtype]), m,
                                         ys, int(mode), bs, _stream_ptr(ctx.device)))
        return [o.reshape(*lead, o.shape[-1]) for o in outs]

    # ---- fused neighbours of the linears (include/turq.h, "Fused neighbours")

    @staticmethod
    def swiglu(gate: "QMatMul", up: "QMatMul", x: torch.Tensor, mode: Mode = Mode.AUTO,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """silu(x . Wg^T) * (x . Wu^T) (tur's Qwen3MLP, src/models/qwen3.rs:160-166), one launch in
        the integer scheme."""
        ctx = gate.qtensor._ctx
        n, k = gate.qtensor.shape()
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        x2 = x.reshape(-1, k).contiguous()
        _check_operand(x2, "x", ctx.device, (torch.float32, torch.bfloat16))
        m = x2.shape[0]
        if out is not None:
            _check_operand(out, "out", ctx.device, (torch.float32,))
        y = out if out is not None else torch.empty((m, n), dtype=torch.float32, device=x2.device)
        ctx.check(_lib.load().turq_qmatmul_swiglu(ctx.handle, gate.qtensor._h, up.qtensor._h, x2.data_ptr(),
                                                  int(_TORCH_TO_GGML[x2.dtype]), m, y.data_ptr(), int(mode), _stream_ptr(ctx.device)))
        return y.reshape(*x.shape[:-1], n)

    @staticmethod
    def rmsnorm_forward_multi(mms: Sequence["QMatMul"], x: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                              biases: Optional[Sequence[Optional[torch.Tensor]]] = None, mode: Mode = Mode.AUTO,
                              return_normed: bool = False):
        """y_i = rmsnorm(x; weight, eps) . W_i^T for linears that share the normalised input
        (ln1 -> attn_q|k|v, ln2 -> ffn_gate|up: src/models/qwen3.rs:633-638). Returns the outputs,
        and the normalised rows too with return_normed."""
        ctx = mms[0].qtensor._ctx
        k = mms[0].qtensor.shape()[1]
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        x2 = x.reshape(-1, k).contiguous()
        _check_operand(x2, "x", ctx.device, (torch.float32, torch.bfloat16))
        _check_operand(norm_weight, "norm_weight", ctx.device, (torch.float32,))
        if norm_weight.numel() != k:
            raise TurqError(2, f"norm weight has {norm_weight.numel()} elements, the linears {k} in-features")
        m, n = x2.shape[0], len(mms)
        outs = [torch.empty((m, mm.qtensor.shape()[0]), dtype=torch.float32, device=x2.device) for mm in mms]
        h = torch.empty((m, k), dtype=torch.float32, device=x2.device) if return_normed else None
        arr = ctypes.c_void_p * n
        bs = None
        if biases is not None:
            for i, b in enumerate(biases):
                if b is not None:
                    _check_operand(b, f"biases[{i}]", ctx.device, (torch.float32,))
            bs = arr(*[b.data_ptr() if b is not None else None for b in biases])
        ctx.check(_lib.load().turq_rmsnorm_qmatmul_multi(
            ctx.handle, n, arr(*[mm.qtensor._h for mm in mms]), x2.data_ptr(), int(_TORCH_TO_GGML[x2.dtype]), m,
            norm_weight.data_ptr(), float(eps), h.data_ptr() if h is not None else None, arr(*[o.data_ptr() for o in outs]),
            int(mode), bs, _stream_ptr(ctx.device)))
        lead = tuple(x.shape[:-1])
        outs = [o.reshape(*lead, o.shape[-1]) for o in outs]
        return (outs, h.reshape(*lead, k)) if return_normed else outs

    def lm_head_topk(self, x: torch.Tensor, k: int = 1, id_offset: int = 0, mode: Optional[Mode] = None,
                     logits_out: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
        """The k best (logit, token id) pairs per row of x . W^T, best first, ties to the lower id
        (greedy decoding: k = 1). tur samples from the last position's logits
        (src/backend/engine.rs:528-529, 810-824)."""
        qt = self.qtensor
        ctx = qt._ctx
        n, kk = qt.shape()
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        x2 = x.reshape(-1, kk).contiguous()
        _check_operand(x2, "x", ctx.device, (torch.float32, torch.bfloat16))
        m = x2.shape[0]
        vals = torch.empty((m, k), dtype=torch.float32, device=x2.device)
        ids = torch.empty((m, k), dtype=torch.int32, device=x2.device)
        if logits_out is not None:
            _check_operand(logits_out, "logits_out", ctx.device, (torch.float32,))
        ctx.check(_lib.load().turq_lm_head_topk(ctx.handle, qt._h, x2.data_ptr(), int(_TORCH_TO_GGML[x2.dtype]), m, k, id_offset,
                                                vals.data_ptr(), ids.data_ptr(),
                                                logits_out.data_ptr() if logits_out is not None else None,
                                                int(self.mode if mode is None else mode), _stream_ptr(ctx.device)))
        return vals, ids


class HostCall:
    """Linears bound to their page-locked host buffers (include/turq.h, turq_host_call_*): the
    caller rewrites `x` in place and calls `run()` token after token; results appear in `outs`.
    One graph launch and one wait on the call's completion word per run. Integer scheme, 1..64
    rows, no bias."""

    def __init__(self, mms: Sequence["QMatMul"], x: torch.Tensor, outs: Optional[Sequence[torch.Tensor]] = None):
        lib = _lib.load()
        self._ctx = mms[0].qtensor._ctx
        k = mms[0].qtensor.shape()[1]
        if x.is_cuda or x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2 or x.shape[1] != k or not x.is_pinned():
            raise TurqError(1, "a bound host call needs a page-locked, contiguous f32 host matrix [m, in-features]")
        m = x.shape[0]
        if outs is None:
            outs = [torch.empty((m, mm.qtensor.shape()[0]), dtype=torch.float32).pin_memory() for mm in mms]
        for o, mm in zip(outs, mms):
            if o.is_cuda or o.dtype != torch.float32 or not o.is_contiguous() or o.numel() != m * mm.qtensor.shape()[0] or not o.is_pinned():
                raise TurqError(1, "outs must be page-locked, contiguous f32 host tensors of m x n elements")
        self.x, self.outs, self._mms = x, list(outs), list(mms)    # keep buffers and weights alive
        n = len(mms)
        arr = ctypes.c_void_p * n
        h = ctypes.c_void_p()
        self._ctx.check(lib.turq_host_call_create(self._ctx.handle, n, arr(*[mm.qtensor._h for mm in mms]), x.data_ptr(), m,
                                                  arr(*[o.data_ptr() for o in self.outs]), ctypes.byref(h)))
        self._h = h
        self._run = lib.turq_host_call_run

    def run(self) -> list[torch.Tensor]:
        st = self._run(self._h)
        if st != 0:
            self._ctx.check(st)
        return self.outs

    __call__ = run

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            _lib.load().turq_host_call_destroy(h)

    __del__ = close


def topk(vals: torch.Tensor, k: int, ids: Optional[torch.Tensor] = None, id_offset: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """k largest per row of vals [m, n] (f32, CUDA) with their ids (positions + id_offset, or the
    given int32 ids [m, n]): best first, ties to the lower id."""
    ctx = context(vals.device)
    _check_operand(vals, "vals", ctx.device, (torch.float32,))
    if ids is not None:
        _check_operand(ids, "ids", ctx.device, (torch.int32,))
    m, n = vals.shape
    ov = torch.empty((m, k), dtype=torch.float32, device=vals.device)
    oi = torch.empty((m, k), dtype=torch.int32, device=vals.device)
    ctx.check(_lib.load().turq_topk(ctx.handle, vals.data_ptr(), ids.data_ptr() if ids is not None else None, m, n, k, id_offset,
                                    ov.data_ptr(), oi.data_ptr(), _stream_ptr(ctx.device)))
    return ov, oi
