"""Megatron-style tensor parallelism for the quantized linear stack (one process per GPU).

tur itself is single-device (no collective anywhere in the reference); this module is the
multi-GPU extension of its linear layers for models whose shapes shard naturally:
  column-parallel (attn_q/k/v, ffn_gate/up, output head): rank r keeps a contiguous run of
      weight rows - GGUF rows are independent block runs, so the shard is a byte slice;
  row-parallel (attn_output, ffn_down): rank r keeps a run of whole blocks of every row and
      multiplies it with its slice of the activation columns; partial results are summed
      with an all-reduce over NCCL (NVLink / NVSwitch).
Sharding happens on the wire-format bytes before upload, so each GPU only ever holds its
shard. The partition arithmetic is plain integer work and is shared by the CUDA path and the
CPU (gloo) tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np

from .workloads import BLOCK, Weight


def split_units(units: int, tp: int) -> list[tuple[int, int]]:
    """Splits `units` into tp contiguous runs whose sizes differ by at most one (larger runs
    first): 100 units over 8 ranks -> 13,13,13,13,12,12,12,12. Returns (start, count)."""
    if tp <= 0 or units < tp:
        raise ValueError(f"cannot split {units} units over {tp} ranks")
    base, extra = divmod(units, tp)
    out, start = [], 0
    for r in range(tp):
        n = base + (1 if r < extra else 0)
        out.append((start, n))
        start += n
    return out


@dataclass(frozen=True)
class Shard:
    """What rank `rank` of `tp` keeps of one weight [n, k]."""
    rows: tuple[int, int]   # (row0, count)
    cols: tuple[int, int]   # (col0, count)
    parallel: str           # "column" | "row"
    unit: int = 16          # granule the split was made in (rows for "column", columns for "row")

    @property
    def shape(self) -> tuple[int, int]:
        return self.rows[1], self.cols[1]


def shard_of(w: Weight, tp: int, rank: int, row_unit: int = 16) -> Shard:
    """Column-parallel weights split their rows in multiples of `row_unit` (head_dim for
    attention projections, 256 for ffn_gate/up so that the shards line up with ffn_down's
    blocks); row-parallel weights split their columns in whole blocks."""
    if w.parallel == "column":
        if w.n % row_unit:
            raise ValueError(f"{w.name}: {w.n} rows are not a multiple of the split unit {row_unit}")
        s, c = split_units(w.n // row_unit, tp)[rank]
        return Shard((s * row_unit, c * row_unit), (0, w.k), "column", row_unit)
    be = BLOCK[w.dtype][0]
    unit = max(be, row_unit if row_unit % be == 0 else be)
    if w.k % unit:
        raise ValueError(f"{w.name}: {w.k} columns are not a multiple of the split unit {unit}")
    s, c = split_units(w.k // unit, tp)[rank]
    return Shard((0, w.n), (s * unit, c * unit), "row", unit)


def shard_blocks(blocks, w: Weight, sh: Shard):
    """Wire-format bytes [n, row_bytes] of the full weight (numpy array or torch uint8 tensor,
    host or device) -> contiguous bytes of the shard, same container type."""
    be, bb = BLOCK[w.dtype]
    full = blocks.reshape(w.n, (w.k // be) * bb)
    if sh.parallel == "column":
        part = full[sh.rows[0]: sh.rows[0] + sh.rows[1]]
    else:
        b0, nb = sh.cols[0] // be, sh.cols[1] // be
        part = full[:, b0 * bb: (b0 + nb) * bb]
    return part.contiguous() if hasattr(part, "contiguous") else np.ascontiguousarray(part)


class TPLinear:
    """One sharded linear. `matmul(x_local) -> y_local` is the per-rank product
    (tur_b200.QMatMul.forward on a GPU; the tests substitute a CPU stand-in), `group` a
    torch.distributed process group (None = default)."""

    def __init__(self, w: Weight, shard: Shard, matmul: Callable, group=None, gather_output: bool = False):
        self.w, self.shard, self.matmul, self.group, self.gather_output = w, shard, matmul, group, gather_output

    def forward(self, x):
        """Column-parallel: x is the full activation, returns this rank's output columns (or
        all of them with gather_output). Row-parallel: x is this rank's activation columns,
        returns the full, summed output on every rank."""
        import torch.distributed as dist
        y = self.matmul(x)
        if self.shard.parallel == "row":
            if dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            return y
        if self.gather_output and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            return gather_columns(y, self.w.n, dist.get_world_size(self.group), self.shard.unit, self.group)
        return y

    __call__ = forward


def gather_columns(y_local, n_total: int, tp: int, row_unit: int, group=None):
    """All-gather of column-parallel outputs with possibly uneven shard widths: pads to the
    widest shard, gathers, and drops the padding."""
    import torch
    import torch.distributed as dist
    parts = split_units(n_total // row_unit, tp)
    widest = max(c for _, c in parts) * row_unit
    m = y_local.shape[0]
    buf = torch.zeros((m, widest), dtype=y_local.dtype, device=y_local.device)
    buf[:, : y_local.shape[1]] = y_local
    out = [torch.empty_like(buf) for _ in range(tp)]
    dist.all_gather(out, buf, group=group)
    return torch.cat([o[:, : c * row_unit] for o, (_, c) in zip(out, parts)], dim=1)


class TPGroup:
    """The ranks of one tensor-parallel group (one process per GPU on one node), exchanging
    through peer memory with the library's own kernels (include/turq.h, turq_tp_*): all-reduce
    behind the row-parallel linears, all-gather behind the column-parallel head. No NCCL call is
    made after construction, so a whole sharded pass can be captured in a CUDA graph.

    Construction is collective: every rank exports a handle and receives everybody's through
    `process_group` (torch.distributed, any backend). `loopback=True` builds a single-process
    group whose other ranks are local stand-ins (tests)."""

    def __init__(self, rank: int, world: int, max_bytes: int, ctx=None, process_group=None, loopback: bool = False):
        import ctypes
        import torch
        from . import _lib
        from .quantized import context
        self._lib, self._ct = _lib.load(), ctypes
        self.ctx = ctx or context()
        self.rank, self.world = rank, world
        h = ctypes.c_void_p()
        self.ctx.check(self._lib.turq_tp_create(self.ctx.handle, rank, world, max_bytes, ctypes.byref(h)))
        self._h = h
        if world == 1:
            return
        if loopback:
            self.ctx.check(self._lib.turq_tp_connect_loopback(h))
            return
        import torch.distributed as dist
        blob = (ctypes.c_uint8 * 64)()
        self.ctx.check(self._lib.turq_tp_export(h, blob))
        mine = bytes(blob)
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=process_group)
        joined = (ctypes.c_uint8 * (64 * world)).from_buffer_copy(b"".join(everyone))
        self.ctx.check(self._lib.turq_tp_connect(h, joined))
        dist.barrier(group=process_group)
        torch.cuda.synchronize()

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.turq_tp_destroy(h)

    __del__ = close

    def _stream(self):
        import torch
        return self._ct.c_void_p(torch.cuda.current_stream(self.ctx.device).cuda_stream)

    def set_wait_limit(self, cycles: int) -> None:
        self.ctx.check(self._lib.turq_tp_set_wait_limit(self._h, cycles))

    def set_fuse_limit(self, nbytes: int) -> None:
        """Largest result the row-parallel matmul exchanges inside its own kernel (0: never)."""
        self.ctx.check(self._lib.turq_tp_set_fuse_limit(self._h, nbytes))

    def set_twoshot_limit(self, nbytes: int) -> None:
        """Smallest result exchanged as reduce-scatter + gather (three or more ranks)."""
        self.ctx.check(self._lib.turq_tp_set_twoshot_limit(self._h, nbytes))

    def set_chunk_rows(self, rows: int) -> None:
        """Rows per chunk of a prefill-sized row-parallel product (0: default)."""
        self.ctx.check(self._lib.turq_tp_set_chunk_rows(self._h, rows))

    def reset(self) -> None:
        self.ctx.check(self._lib.turq_tp_reset(self._h))

    def allreduce(self, x, out=None):
        """Sum over the ranks, added in rank order on every rank (f32, contiguous)."""
        import torch
        out = torch.empty_like(x) if out is None else out
        self.ctx.check(self._lib.turq_tp_allreduce(self._h, self._ct.c_void_p(x.data_ptr()), self._ct.c_void_p(out.data_ptr()),
                                                   x.numel(), self._stream()))
        return out

    def allgather(self, x, widths: Sequence[int], out=None):
        """x [m, widths[rank]] -> [m, sum(widths)] on every rank."""
        import torch
        m = x.shape[0]
        out = torch.empty((m, sum(widths)), dtype=torch.float32, device=x.device) if out is None else out
        w = (self._ct.c_int64 * self.world)(*widths)
        self.ctx.check(self._lib.turq_tp_allgather(self._h, self._ct.c_void_p(x.data_ptr()), m, w, self._ct.c_void_p(out.data_ptr()),
                                                   self._stream()))
        return out

    def qmatmul_rowparallel(self, mm, x, bias=None, mode=None, out=None):
        """Row-parallel linear: this rank's column range of the weight times its slice of the
        activations, summed over the ranks (+ bias). mm is a tur_b200.QMatMul on the shard."""
        import torch
        from .quantized import _TORCH_TO_GGML, Mode
        qt = mm.qtensor
        n, k = qt.shape()
        x2 = x.reshape(-1, k).contiguous()
        m = x2.shape[0]
        out = torch.empty((m, n), dtype=torch.float32, device=x.device) if out is None else out
        mode = (mm.mode if mode is None else mode)
        self.ctx.check(self._lib.turq_qmatmul_rowparallel(
            self._h, qt._h, self._ct.c_void_p(x2.data_ptr()), int(_TORCH_TO_GGML[x2.dtype]), m, self._ct.c_void_p(out.data_ptr()),
            int(mode), self._ct.c_void_p(bias.data_ptr()) if bias is not None else None, self._stream()))
        return out

    def qmatmul_gather(self, mm, x, widths: Sequence[int], bias=None, mode=None, out=None):
        """Column-parallel linear with gathered output (the vocabulary-sharded head): this rank's
        rows of the weight times the full activations, every rank's columns on every rank."""
        import torch
        from .quantized import _TORCH_TO_GGML
        qt = mm.qtensor
        n, k = qt.shape()
        x2 = x.reshape(-1, k).contiguous()
        m = x2.shape[0]
        out = torch.empty((m, sum(widths)), dtype=torch.float32, device=x.device) if out is None else out
        w = (self._ct.c_int64 * self.world)(*widths)
        self.ctx.check(self._lib.turq_qmatmul_gather(
            self._h, qt._h, x2.data_ptr(), int(_TORCH_TO_GGML[x2.dtype]), m, w, out.data_ptr(), int(mm.mode if mode is None else mode),
            bias.data_ptr() if bias is not None else None, self._stream()))
        return out

    def loopback_fill(self, peer: int, data=None, signal=True) -> None:
        """Tests: play rank `peer`'s part for the next call: its data and, with `signal`, its flags
        (an integer k > 1: it has arrived at the next k calls already)."""
        ptr = self._ct.c_void_p(data.data_ptr()) if data is not None else None
        self.ctx.check(self._lib.turq_tp_loopback_fill(self._h, peer, ptr, data.numel() if data is not None else 0,
                                                       int(signal), self._stream()))


def row_unit_for(w: Weight, head_dim: Optional[int] = None) -> int:
    """Split unit of a weight inside a decoder layer: whole heads for attention projections
    (and the matching column blocks of attn_output), 256-wide blocks for the MLP."""
    if w.name in ("attn_q", "attn_k", "attn_v", "attn_output") and head_dim:
        return head_dim
    if w.name in ("ffn_gate", "ffn_up", "ffn_down"):
        return 256
    return 16
