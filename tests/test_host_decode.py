"""The device layout code run on the CPU: layout.h's repack map and decode.cuh's per-lane tile
decoder are `__host__ __device__`, so a host program (compiled with nvcc, no GPU needed) can
push the golden GGUF blocks through exactly the code the dequantize kernel executes and compare
with gguf-py's values bit for bit - one block per row (ragged row-tiles) and several blocks per
row (the K-tile walk)."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TYPES = list(oracle.WEIGHT_TYPES)


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc) and not shutil.which("nvcc"):
        pytest.skip("nvcc not available")
    exe = str(tmp_path_factory.mktemp("hostdecode") / "host_decode_check")
    subprocess.run([nvcc, "-O1", "-std=c++17", "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "tur_b200", "csrc"),
                    "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "host_decode_check.cu"), "-o", exe],
                   check=True)
    return exe


def run_case(checker, tmp_path, dt, blocks, want, n, k):
    bf, ff = str(tmp_path / "blocks.bin"), str(tmp_path / "f32.bin")
    np.ascontiguousarray(blocks, dtype=np.uint8).tofile(bf)
    np.ascontiguousarray(want, dtype=np.float32).tofile(ff)
    r = subprocess.run([checker, str(dt), str(n), str(k), bf, ff], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.parametrize("dt", TYPES, ids=[oracle.NAMES[t] for t in TYPES])
def test_device_decoder_on_cpu_matches_gguf_golden(checker, tmp_path, golden_dir, dt):
    g = np.load(os.path.join(golden_dir, "gguf_dequantize.npz"))
    name = oracle.NAMES[dt]
    blocks, want = g[f"{name}_blocks"], g[f"{name}_f32"]
    nb, be = blocks.shape[0], oracle.block_elems(dt)
    # one block per row: 133 / 49 / 51 rows, so the last row-tile is ragged
    run_case(checker, tmp_path, dt, blocks, want, nb, be)
    # several blocks per row: rows of 7 (or 19 for Q8_0) consecutive blocks
    per_row = 19 if dt == oracle.Q8_0 else 7
    rows = nb // per_row
    run_case(checker, tmp_path, dt, blocks[: rows * per_row], want[: rows * per_row], rows, per_row * be)


@pytest.mark.parametrize("dt", TYPES, ids=[oracle.NAMES[t] for t in TYPES])
def test_device_decoder_on_cpu_matches_oracle_on_quantized_weights(checker, tmp_path, dt):
    rng = np.random.default_rng(299792458 + dt)
    n, k = 37, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    blocks = oracle.quantize(dt, w)
    run_case(checker, tmp_path, dt, blocks, oracle.dequantize(dt, blocks, k), n, k)
