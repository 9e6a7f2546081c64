"""Shapes of the quantized-linear stacks the benchmark configs name (out x in per weight).

Each workload is a decoder's per-layer linear set as tur builds it
(src/models/qwen3.rs:153-155 MLP, :212-215 attention; src/models/granite_41.rs:142-144,
:192-195) with the per-weight GGUF types of the named quantization mix: in the *_K_M mixes
`attn_v` and `ffn_down` (and the output head) are Q6_K, the rest Q4_K or Q5_K.
"""
from __future__ import annotations

from dataclasses import dataclass

Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}
SEED = 299792458  # tur's default seed (src/backend/engine.rs:60)


@dataclass(frozen=True)
class Weight:
    name: str       # GGUF tensor stem: attn_q, attn_k, attn_v, attn_output, ffn_gate, ffn_up, ffn_down, output
    n: int          # out features (rows)
    k: int          # in features (cols)
    dtype: int
    source: str     # which activation feeds it: "hidden", "attn", "inter"
    parallel: str   # tensor-parallel split: "column" (split n) or "row" (split k)

    @property
    def nbytes(self) -> int:
        be, bb = BLOCK[self.dtype]
        return self.n * (self.k // be) * bb


@dataclass(frozen=True)
class Workload:
    name: str
    description: str
    hidden: int
    layers: int
    per_layer: tuple
    head: Weight | None

    def layer_bytes(self) -> int:
        return sum(w.nbytes for w in self.per_layer)

    def total_bytes(self) -> int:
        return self.layers * self.layer_bytes() + (self.head.nbytes if self.head else 0)

    def flops_per_row(self) -> int:
        per = sum(2 * w.n * w.k for w in self.per_layer) * self.layers
        return per + (2 * self.head.n * self.head.k if self.head else 0)


def _decoder(hidden, q_out, kv_out, inter, main, alt):
    return (
        Weight("attn_q", q_out, hidden, main, "hidden", "column"),
        Weight("attn_k", kv_out, hidden, main, "hidden", "column"),
        Weight("attn_v", kv_out, hidden, alt, "hidden", "column"),
        Weight("attn_output", hidden, q_out, main, "attn", "row"),
        Weight("ffn_gate", inter, hidden, main, "hidden", "column"),
        Weight("ffn_up", inter, hidden, main, "hidden", "column"),
        Weight("ffn_down", hidden, inter, alt, "inter", "row"),
    )


def _mk(name, desc, hidden, q_out, kv_out, inter, layers, main, alt, vocab=None):
    head = Weight("output", vocab, hidden, Q6_K if main != Q8_0 else Q8_0, "hidden", "column") if vocab else None
    return Workload(name, desc, hidden, layers, _decoder(hidden, q_out, kv_out, inter, main, alt), head)


WORKLOADS = {
    "cfg1": _mk("cfg1", "Qwen3-0.6B linear stack, Q8_0", 1024, 2048, 1024, 3072, 28, Q8_0, Q8_0),
    "cfg2": _mk("cfg2", "Qwen3-8B linear stack, Q4_K_M (+ Q6_K lm_head)", 4096, 4096, 1024, 12288, 36, Q4_K, Q6_K, 151936),
    "cfg3-q5": _mk("cfg3-q5", "Qwen3-8B linear stack, Q5_K_M", 4096, 4096, 1024, 12288, 36, Q5_K, Q6_K, 151936),
    "cfg4-q5": _mk("cfg4-q5", "3B dense decoder linear stack, Q5_K_M", 2560, 2560, 640, 8192, 40, Q5_K, Q6_K),
    "cfg4-q8": _mk("cfg4-q8", "3B dense decoder linear stack, Q8_0", 2560, 2560, 640, 8192, 40, Q8_0, Q8_0),
    "cfg5": _mk("cfg5", "Qwen3-32B linear stack, Q4_K_M (+ Q6_K lm_head)", 5120, 8192, 1024, 25600, 64, Q4_K, Q6_K, 151936),
}


def random_blocks(dtype: int, n: int, k: int, seed: int, device):
    """Valid wire blocks with plausible scales, generated on the GPU as a flat uint8 tensor.
    Timing input only: the quantized values are uniform bytes, not a quantized Gaussian."""
    import torch
    be, bb = BLOCK[dtype]
    g = torch.Generator(device=device).manual_seed(seed)
    nb = n * (k // be)
    raw = torch.randint(0, 256, (nb, bb), dtype=torch.uint8, device=device, generator=g)
    scale = (torch.rand((nb,), device=device, generator=g) * 0.004 + 0.0005).to(torch.float16).view(torch.uint8).reshape(nb, 2)
    if dtype == Q6_K:
        raw[:, 208:210] = scale
    else:
        raw[:, 0:2] = scale
        if dtype in (Q4_K, Q5_K):
            raw[:, 2:4] = scale
    return raw.reshape(-1)


def quantized_blocks(dtype: int, n: int, k: int, seed: int, device):
    """Seeded N(0, 0.02) weights [n, k] quantized on the GPU to wire blocks of `dtype` (flat uint8
    tensor): the value distribution the benchmark configurations prescribe, made by the library's
    own weight quantizer (turq_quantize_weights), in slabs of rows so that the f32 source of a
    large vocabulary matrix never has to exist as a whole."""
    import torch
    from .quantized import GgmlDType, quantize_weights
    g = torch.Generator(device=device).manual_seed(seed)
    rows_per_slab = max(16, (1 << 26) // k)
    parts = []
    for r0 in range(0, n, rows_per_slab):
        r = min(rows_per_slab, n - r0)
        w = torch.randn((r, k), device=device, generator=g, dtype=torch.float32) * 0.02
        parts.append(quantize_weights(w, GgmlDType(dtype)).reshape(-1))
    return torch.cat(parts) if len(parts) > 1 else parts[0]

