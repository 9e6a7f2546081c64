"""Mirror of tur's quantized linear layer (src/models/layers/linear.rs).

`LinearX.Quantized{qmatmul, bias}` keeps the GGUF weight quantized on the device and runs
`QMatMul::forward`, then adds the optional f32 bias (linear.rs:19-32); `linear(in_dim,
out_dim, vb)` builds it from a var-builder that hands out QTensors (linear.rs:50-70). Here
the bias add is fused into the matmul kernel's epilogue.
"""
from __future__ import annotations

from typing import Optional, Protocol

import torch

from .quantized import Mode, QMatMul, QTensor, TurqError


class QVarBuilderLike(Protocol):
    """The part of src/weights/gguf_varbuilder.rs a linear layer needs."""

    def get(self, shape, name: str) -> QTensor: ...
    def contains_key(self, name: str) -> bool: ...


class LinearX:
    """The `Quantized` arm of tur's LinearX enum."""

    def __init__(self, qmatmul: QMatMul, bias: Optional[torch.Tensor] = None):
        self.qmatmul = qmatmul
        self.bias = bias

    def forward(self, x: torch.Tensor, mode: Optional[Mode] = None) -> torch.Tensor:
        return self.qmatmul.forward(x, bias=self.bias, mode=mode)

    __call__ = forward

    def __repr__(self) -> str:
        return "LinearX::Quantized"


def linear(in_dim: int, out_dim: int, vb: QVarBuilderLike) -> LinearX:
    """linear.rs:50-70: weight `(out_dim, in_dim)` stays quantized; a `bias` tensor, when the
    file has one, is dequantized to f32 once."""
    qweight = vb.get((out_dim, in_dim), "weight")
    if tuple(qweight.shape()) != (out_dim, in_dim):
        raise TurqError(2, f"shape mismatch for weight, got {qweight.shape()}, expected {(out_dim, in_dim)}")
    bias = None
    if vb.contains_key("bias"):
        b = vb.get(out_dim, "bias")
        bias = b.dequantize().reshape(out_dim) if hasattr(b, "dequantize") else b
    return LinearX(QMatMul.from_arc(qweight), bias)
