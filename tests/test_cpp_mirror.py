"""The C++ host-side mirror (include/turq.hpp) compiles against the C ABI, links with
libturq.so, and reports the no-GPU case as an error instead of falling back."""
import os
import subprocess
import tempfile

import pytest
import torch

from tur_b200.build import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include <cstdio>
#include <vector>
#include "turq.hpp"
int main() {
  std::printf("Q4K %d/%d Q6K %d/%d\n", turq::block_size(turq::GgmlDType::Q4K), turq::type_size(turq::GgmlDType::Q4K),
              turq::block_size(turq::GgmlDType::Q6K), turq::type_size(turq::GgmlDType::Q6K));
  try {
    auto ctx = std::make_shared<turq::Context>(0);
    std::vector<unsigned char> blocks(16 * 144, 0);
    auto w = turq::QTensor::from_host(ctx, turq::GgmlDType::Q4K, 16, 256, blocks.data(), blocks.size());
    auto mm = turq::QMatMul::from_arc(w);
    std::vector<float> x(256, 1.0f);
    auto y = mm.forward_host(x.data(), 1);
    std::printf("gpu ok rows=%zu y0=%g\n", y.size(), y[0]);
  } catch (const turq::Error& e) {
    std::printf("error status=%d %s\n", e.status, e.what());
  }
  return 0;
}
"""


def test_cpp_mirror_compiles_links_and_reports_errors():
    lib = build()
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "t.cpp"), os.path.join(d, "t")
        open(src, "w").write(PROGRAM)
        libdir = os.path.dirname(lib)
        subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), src, "-o", exe, "-L", libdir, "-lturq",
                        f"-Wl,-rpath,{libdir}", "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64"], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    assert "Q4K 256/144 Q6K 256/210" in out
    if torch.cuda.is_available():
        assert "gpu ok rows=16 y0=0" in out
    else:
        assert "error status=8" in out
