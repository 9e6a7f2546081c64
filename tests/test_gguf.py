"""GGUF container reader and the lazy var-builder (tur: src/weights/gguf_varbuilder.rs):
files are written with the gguf python package's writer, blocks come from the CPU oracle."""
import io
import os

import numpy as np
import pytest
import torch

import oracle
from tur_b200.gguf import Content, GgufError, VarBuilder

K, N = 512, 48


@pytest.fixture(scope="module")
def gguf_file(tmp_path_factory):
    import gguf
    from gguf.constants import GGMLQuantizationType as T
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    rng = np.random.default_rng(3)
    w = gguf.GGUFWriter(path, "qwen3")
    w.add_uint32("qwen3.block_count", 1)
    w.add_string("general.name", "tiny")
    tensors = {}
    for name, dt, gt, n in (("blk.0.attn_q.weight", oracle.Q4_K, T.Q4_K, N), ("blk.0.attn_v.weight", oracle.Q6_K, T.Q6_K, 16),
                            ("blk.0.ffn_up.weight", oracle.Q5_K, T.Q5_K, 32), ("output.weight", oracle.Q8_0, T.Q8_0, 40)):
        f32 = (rng.standard_normal((n, K)) * 0.02).astype(np.float32)
        blocks = oracle.quantize(dt, f32)
        tensors[name] = (dt, n, blocks)
        w.add_tensor(name, blocks, raw_shape=blocks.shape, raw_dtype=gt)
    norm = rng.standard_normal(K).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    w.add_tensor("blk.0.attn_norm.weight", norm)
    w.add_tensor("blk.0.attn_q.bias", bias)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, tensors, norm, bias


def test_header_and_tensor_table(gguf_file):
    path, tensors, norm, _ = gguf_file
    with open(path, "rb") as f:
        c = Content.read(f)
        assert c.metadata["general.name"] == "tiny" and c.metadata["qwen3.block_count"] == 1
        assert set(c.tensor_infos) == set(tensors) | {"blk.0.attn_norm.weight", "blk.0.attn_q.bias"}
        for name, (dt, n, blocks) in tensors.items():
            info, raw = c.tensor_bytes(f, name)
            assert info.shape == (n, K) and info.ggml_dtype == dt
            assert np.array_equal(raw, blocks.reshape(-1))
        info, raw = c.tensor_bytes(f, "blk.0.attn_norm.weight")
        assert info.shape == (K,) and np.array_equal(raw.view(np.float32), norm)
        with pytest.raises(GgufError):
            c.tensor_bytes(f, "blk.9.missing.weight")


def test_var_builder_names_and_shapes(gguf_file):
    path, tensors, _, _ = gguf_file
    vb = VarBuilder.from_gguf(path)
    blk = vb.pp("blk").pp(0)
    assert blk.path("attn_q.weight") == "blk.0.attn_q.weight"
    assert blk.pp("attn_q").contains_key("weight") and not blk.pp("attn_k").contains_key("weight")
    assert blk.pp("attn_q").tensor_shape("weight") == [N, K]
    assert sorted(vb.all_keys()) == sorted(list(tensors) + ["blk.0.attn_norm.weight", "blk.0.attn_q.bias"])


def test_rejects_files_that_are_not_gguf():
    with pytest.raises(GgufError):
        Content.read(io.BytesIO(b"GGML" + bytes(64)))
    with pytest.raises(GgufError):
        Content.read(io.BytesIO(b"GGUF" + (99).to_bytes(4, "little") + bytes(64)))


@pytest.mark.gpu
def test_tensors_go_to_the_gpu_and_build_a_linear(gguf_file):
    from tur_b200 import Mode, QTensor, linear
    path, tensors, norm, bias = gguf_file
    vb = VarBuilder.from_gguf(path)
    for name, (dt, n, blocks) in tensors.items():
        stem, _, leaf = name.rpartition(".")
        sub = vb
        for part in stem.split("."):
            sub = sub.pp(part)
        t = sub.get((n, K), leaf)
        assert isinstance(t, QTensor) and t.shape() == (n, K)
        assert np.array_equal(t.dequantize().cpu().numpy(), oracle.dequantize(dt, blocks, K))
        assert sub.get((n, K), leaf) is t                     # one-entry cache
        with pytest.raises(GgufError):
            sub.get((n + 1, K), leaf)
    got_norm = vb.pp("blk").pp(0).pp("attn_norm").get(K, "weight").dequantize().cpu().numpy()
    assert np.array_equal(got_norm, norm)
    # tur's linear(): quantized weight + f32 bias from the same prefix (src/models/layers/linear.rs:50-70)
    lin = linear(K, N, vb.pp("blk").pp(0).pp("attn_q"))
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, K)).astype(np.float32)
    y = lin(torch.from_numpy(x).cuda(), mode=Mode.INT8_ACT).cpu().numpy()
    dt, n, blocks = tensors["blk.0.attn_q.weight"]
    assert oracle.rel_fro(y, oracle.qmatmul(dt, blocks, n, K, x) + bias) < 1e-5
