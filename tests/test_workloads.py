"""Byte and flop counts of the benchmark workloads: the throughput metrics are computed from
these, so they are pinned to the GGUF block sizes (gguf-py constants.py:4239-4245) and to the
shapes the benchmark configurations name."""
import pytest

from tur_b200.workloads import BLOCK, Q4_K, Q5_K, Q6_K, Q8_0, WORKLOADS


def test_block_geometry_is_ggufs():
    assert BLOCK == {Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}


@pytest.mark.parametrize("name,layers,layer_bytes,head_bytes", [
    ("cfg1", 28, 16_711_680, None),
    ("cfg2", 36, 122_585_088, 510_504_960),
    ("cfg3-q5", 36, 139_886_592, 510_504_960),
    ("cfg4-q5", 40, 57_520_640, None),
    ("cfg4-q8", 40, 84_254_720, None),
    ("cfg5", 64, 309_411_840, 638_131_200),
])
def test_layer_and_head_bytes(name, layers, layer_bytes, head_bytes):
    wl = WORKLOADS[name]
    assert wl.layers == layers
    assert wl.layer_bytes() == layer_bytes
    assert (wl.head.nbytes if wl.head else None) == head_bytes
    assert wl.total_bytes() == layers * layer_bytes + (head_bytes or 0)


def test_cfg2_weights_are_the_named_mix():
    by = {w.name: w for w in WORKLOADS["cfg2"].per_layer}
    assert (by["attn_q"].n, by["attn_q"].k, by["attn_q"].dtype) == (4096, 4096, Q4_K)
    assert (by["attn_k"].n, by["attn_v"].n) == (1024, 1024)
    assert by["attn_v"].dtype == Q6_K and by["ffn_down"].dtype == Q6_K
    assert (by["ffn_gate"].n, by["ffn_up"].n, by["ffn_down"].k) == (12288, 12288, 12288)
    assert {w.parallel for w in by.values() if w.name in ("attn_output", "ffn_down")} == {"row"}
    assert WORKLOADS["cfg2"].head.dtype == Q6_K and WORKLOADS["cfg2"].head.n == 151936


def test_flops_per_row():
    wl = WORKLOADS["cfg2"]
    per_layer = 2 * sum(w.n * w.k for w in wl.per_layer)
    assert per_layer * 512 == 197_568_495_616          # 197.57 GFLOP per layer at M = 512
    assert wl.flops_per_row() == 36 * per_layer + 2 * 151936 * 4096
