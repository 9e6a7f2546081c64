"""GGUF container reader and the lazy tensor provider tur builds its layers from.

Mirrors what tur uses of candle's `gguf_file::Content` and its own
`src/weights/gguf_varbuilder.rs`: the header and tensor table are parsed once, a tensor's raw
blocks are read from the file on demand and go straight to the GPU as a `QTensor` (device
fragment tiles), with a one-entry cache and dotted path prefixes (`vb.pp("blk").pp(3)`).
Only host-side byte handling happens here; the file format is the public GGUF v2/v3 layout.
"""
from __future__ import annotations

import struct
import threading
from dataclasses import dataclass
from typing import BinaryIO, Optional, Sequence

import numpy as np
import torch

from .quantized import GgmlDType, QTensor, TurqError, _Context, context

GGUF_MAGIC = b"GGUF"
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9
# elements per block, bytes per block for the tensor types this library can hold
_GEOMETRY = {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple          # outermost dimension first, e.g. (out_features, in_features)
    ggml_dtype: int
    offset: int           # from the start of the data section
    nbytes: int


class GgufError(TurqError):
    def __init__(self, message: str):
        super().__init__(2, message)


def _read(f: BinaryIO, fmt: str):
    size = struct.calcsize(fmt)
    b = f.read(size)
    if len(b) != size:
        raise GgufError("unexpected end of file")
    return struct.unpack(fmt, b)[0]


def _read_string(f: BinaryIO) -> str:
    n = _read(f, "<Q")
    if n > 1 << 24:
        raise GgufError(f"implausible string length {n}")
    return f.read(n).decode("utf-8", errors="replace")


def _read_value(f: BinaryIO, t: int):
    if t in _SCALAR:
        return _read(f, _SCALAR[t])
    if t == _T_STRING:
        return _read_string(f)
    if t == _T_ARRAY:
        et = _read(f, "<I")
        n = _read(f, "<Q")
        return [_read_value(f, et) for _ in range(n)]
    raise GgufError(f"unknown metadata value type {t}")


class Content:
    """Parsed GGUF header: metadata, tensor table, start of the data section
    (candle: gguf_file::Content::read, called at src/weights/gguf_varbuilder.rs:22)."""

    def __init__(self, metadata: dict, tensor_infos: dict, data_offset: int):
        self.metadata = metadata
        self.tensor_infos = tensor_infos
        self.tensor_data_offset = data_offset

    @classmethod
    def read(cls, f: BinaryIO) -> "Content":
        if f.read(4) != GGUF_MAGIC:
            raise GgufError("not a GGUF file (bad magic)")
        version = _read(f, "<I")
        if version not in (2, 3):
            raise GgufError(f"unsupported GGUF version {version}")
        n_tensors = _read(f, "<Q")
        n_kv = _read(f, "<Q")
        metadata = {}
        for _ in range(n_kv):
            key = _read_string(f)
            metadata[key] = _read_value(f, _read(f, "<I"))
        infos = {}
        for _ in range(n_tensors):
            name = _read_string(f)
            n_dims = _read(f, "<I")
            dims = [_read(f, "<Q") for _ in range(n_dims)]      # innermost first in the file
            dt = _read(f, "<I")
            off = _read(f, "<Q")
            shape = tuple(reversed(dims))
            geo = _GEOMETRY.get(dt)
            nbytes = 0
            if geo is not None and dims:
                be, bb = geo
                if dims[0] % be:
                    raise GgufError(f"tensor {name}: inner dimension {dims[0]} is not a multiple of the block size {be}")
                nbytes = int(np.prod(dims, dtype=np.int64)) // be * bb
            infos[name] = TensorInfo(name, shape, dt, off, nbytes)
        align = int(metadata.get("general.alignment", 32))
        pos = f.tell()
        data_offset = (pos + align - 1) // align * align
        return cls(metadata, infos, data_offset)

    def tensor_bytes(self, f: BinaryIO, name: str) -> tuple[TensorInfo, np.ndarray]:
        info = self.tensor_infos.get(name)
        if info is None:
            raise GgufError(f"cannot find tensor info for {name}")
        if info.ggml_dtype not in _GEOMETRY:
            raise TurqError(3, f"tensor {name} has GGML type {info.ggml_dtype}, which this library does not hold")
        f.seek(self.tensor_data_offset + info.offset)
        raw = f.read(info.nbytes)
        if len(raw) != info.nbytes:
            raise GgufError(f"tensor {name}: file ends inside the tensor data")
        return info, np.frombuffer(raw, dtype=np.uint8)

    def tensor(self, f: BinaryIO, name: str, device=None, ctx: Optional[_Context] = None):
        """Reads one tensor's blocks and puts them on the GPU: a `QTensor` for Q8_0 / Q4_K /
        Q5_K / Q6_K, a `DenseTensor` for F32 / F16 / BF16 (norm weights, biases)."""
        info, raw = self.tensor_bytes(f, name)
        if info.ggml_dtype in (0, 1, 30):
            return DenseTensor(info, raw, device)
        rows = int(np.prod(info.shape[:-1], dtype=np.int64)) if len(info.shape) > 1 else 1
        return QTensor.new(raw, GgmlDType(info.ggml_dtype), (rows, info.shape[-1]), device=device, ctx=ctx)


class DenseTensor:
    """An unquantized GGUF tensor (F32 / F16 / BF16); `dequantize()` gives f32 on the device,
    like candle's QTensor::dequantize does for these types (src/models/layers/norm.rs:82-84)."""

    def __init__(self, info: TensorInfo, raw: np.ndarray, device=None):
        self._info = info
        np_dt = {0: np.float32, 1: np.float16, 30: np.uint16}[info.ggml_dtype]
        host = torch.from_numpy(raw.view(np_dt).reshape(info.shape).copy())
        if info.ggml_dtype == 30:
            host = host.view(torch.bfloat16)
        dev = torch.device("cuda", context(device).device) if torch.cuda.is_available() else torch.device("cpu")
        self._t = host.to(dev)

    def shape(self):
        return tuple(self._info.shape)

    def dtype(self) -> GgmlDType:
        return GgmlDType(self._info.ggml_dtype)

    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return self._t.to(out_dtype)


class VarBuilder:
    """tur's QVarBuilder (src/weights/gguf_varbuilder.rs:11-117): lazy tensors by dotted name,
    the file kept open behind a lock, the last tensor cached, shapes checked on `get`."""

    def __init__(self, content: Content, file: BinaryIO, lock: threading.Lock, cache: dict, path: Sequence[str], device):
        self.content, self._file, self._lock, self._cache, self._path, self._device = content, file, lock, cache, list(path), device

    @classmethod
    def from_gguf(cls, p, device=None) -> "VarBuilder":
        f = open(p, "rb")
        return cls(Content.read(f), f, threading.Lock(), {"name": None, "tensor": None}, [], device)

    def pp(self, s) -> "VarBuilder":
        return VarBuilder(self.content, self._file, self._lock, self._cache, self._path + [str(s)], self._device)

    def path(self, tensor_name: str) -> str:
        return ".".join(self._path + [tensor_name]) if self._path else tensor_name

    def get(self, s, name: str):
        shape = tuple(int(d) for d in (s if isinstance(s, (tuple, list)) else (s,)))
        path = self.path(name)
        with self._lock:
            if self._cache["name"] == path:
                t = self._cache["tensor"]
            else:
                t = self.content.tensor(self._file, path, self._device)
                self._cache["name"], self._cache["tensor"] = path, t
        got = tuple(t.shape())
        want = (1,) + shape if isinstance(t, QTensor) and len(shape) == 1 else shape
        if got != tuple(want):
            raise GgufError(f"shape mismatch for {name}, got {got}, expected {shape}")
        return t

    def get_no_shape(self, name: str):
        with self._lock:
            return self.content.tensor(self._file, self.path(name), self._device)

    def device(self):
        return self._device

    def contains_key(self, key: str) -> bool:
        return self.path(key) in self.content.tensor_infos

    def tensor_shape(self, key: str):
        info = self.content.tensor_infos.get(self.path(key))
        return list(info.shape) if info else None

    def all_keys(self) -> list:
        return list(self.content.tensor_infos.keys())
