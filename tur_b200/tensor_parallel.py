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


def row_unit_for(w: Weight, head_dim: Optional[int] = None) -> int:
    """Split unit of a weight inside a decoder layer: whole heads for attention projections
    (and the matching column blocks of attn_output), 256-wide blocks for the MLP."""
    if w.name in ("attn_q", "attn_k", "attn_v", "attn_output") and head_dim:
        return head_dim
    if w.name in ("ffn_gate", "ffn_up", "ffn_down"):
        return 256
    return 16
