"""Host-side launch arithmetic (tur_b200/csrc/launch_plan.h), compiled with g++ and checked on
the CPU: every tile of a weight is owned by exactly one CTA, whole-row-tile splits are what they
claim, the workspace is large enough for the grid, and the GEMM's split-K / tile choices keep
their invariants (at least 8 K blocks per split, independent of the batch size for decode)."""
import ctypes
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = r"""
#include "launch_plan.h"
extern "C" {
void plan_split(int row_tiles, int KU, int slots, int force, int* out) {
  turq::GemvSplit p = turq::plan_gemv_split(row_tiles, KU, slots, force);
  out[0] = p.grid; out[1] = p.split_q; out[2] = p.split_r; out[3] = p.aligned ? 1 : 0;
}
long long split_start(int grid, int q, int r, long long total, int b) {
  turq::GemvSplit p{grid, q, r, false};
  return turq::gemv_split_start(p, total, b);
}
int gemm_bn(long long n, long long m, int sms, int force) { return turq::plan_gemm_bn(n, m, sms, force); }
int gemm_splits(long long n, long long m, long long k, int sms, int force) { return turq::plan_gemm_splits(n, m, k, sms, force); }
}
"""


@pytest.fixture(scope="module")
def plan():
    with tempfile.TemporaryDirectory() as d:
        src, so = os.path.join(d, "shim.cpp"), os.path.join(d, "shim.so")
        open(src, "w").write(SHIM)
        subprocess.run(["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-I", os.path.join(ROOT, "tur_b200", "csrc"),
                        src, "-o", so], check=True)
        lib = ctypes.CDLL(so)
        lib.split_start.restype = ctypes.c_longlong
        lib.split_start.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
        lib.gemm_bn.argtypes = [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_int]
        lib.gemm_splits.argtypes = [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_int]
        yield lib


SLOTS = 296  # two CTAs on each of 148 SMs
# (rows, K tiles per row-tile): the benchmark shapes plus ragged and tiny ones
SHAPES = [(1024, 16), (4096, 16), (5120, 16), (12288, 16), (24576, 16), (4096, 48), (151936, 16), (8192, 20),
          (5120, 32), (5120, 100), (25600, 20), (2560, 10), (640, 10), (2048, 8), (3072, 8), (1, 1), (3, 2),
          (17, 5), (49155, 10), (300, 25), (9500, 1), (4737, 7)]


@pytest.mark.parametrize("force", [-1, 0, 1])
@pytest.mark.parametrize("rows,ku", SHAPES)
def test_every_unit_has_exactly_one_owner(plan, rows, ku, force):
    row_tiles = (rows + 15) // 16
    out = (ctypes.c_int * 4)()
    plan.plan_split(row_tiles, ku, SLOTS, force, out)
    grid, q, r, aligned = out[0], out[1], out[2], out[3]
    total = row_tiles * ku
    assert 1 <= grid <= SLOTS
    starts = [plan.split_start(grid, q, r, total, b) for b in range(grid + 1)]
    assert starts[0] == 0 and starts[-1] == total
    assert all(a <= b for a, b in zip(starts, starts[1:]))
    assert all(b > a for a, b in zip(starts, starts[1:])), "no CTA without work"
    if aligned:
        assert all(s % ku == 0 for s in starts), "whole row-tiles only"
        per = q // ku
        assert per == -(-row_tiles // SLOTS)
    else:
        sizes = [b - a for a, b in zip(starts, starts[1:])]
        assert max(sizes) - min(sizes) <= 1, "even split"
    # hand-over workspace: one flag and one partial-sum slot per CTA, sized for 4 CTAs per SM
    assert grid <= 148 * 4


def test_split_choice_follows_the_stated_rule(plan):
    out = (ctypes.c_int * 4)()
    plan.plan_split(768, 16, SLOTS, -1, out)       # ffn_gate 12288 rows: 3 row-tiles per CTA, 256 CTAs (86 %)
    assert (out[0], out[1], out[3]) == (256, 48, 1)
    plan.plan_split(320, 32, SLOTS, -1, out)       # 5120 x 8192: 160 CTAs would idle 46 % of the slots, large -> even split
    assert out[3] == 0 and out[0] == SLOTS
    plan.plan_split(64, 16, SLOTS, -1, out)        # 1024 rows: small -> whole row-tiles on 64 CTAs
    assert (out[0], out[3]) == (64, 1)


@pytest.mark.parametrize("n,k", [(8192, 5120), (1024, 5120), (5120, 8192), (25600, 5120), (5120, 25600), (2560, 2560),
                                  (640, 2560), (12288, 4096), (4096, 12288), (151936, 4096), (272, 256), (128, 512)])
def test_gemm_split_k_invariants(plan, n, k):
    sms = 148
    decode = {plan.gemm_splits(n, m, k, sms, -1) for m in (17, 32, 48, 64)}
    assert len(decode) == 1, "the split must not depend on the batch size"
    s = decode.pop()
    assert 1 <= s <= 16
    if s > 1:
        assert (k // 64) // s >= 8, "at least 8 K blocks per CTA"
        assert s * ((n + 127) // 128) <= sms, "one wave"
    for m in (65, 512, 4096):
        assert plan.gemm_splits(n, m, k, sms, -1) == 1
    assert plan.gemm_splits(n, 64, k, sms, 0) == 1


def test_gemm_activation_tile_choice(plan):
    sms = 148
    assert plan.gemm_bn(12288, 64, sms, 0) == 64
    assert plan.gemm_bn(12288, 2048, sms, 0) == 256
    assert plan.gemm_bn(4096, 512, sms, 0) == 128      # 32 x 2 tiles: doubling still fits one wave
    assert plan.gemm_bn(2560, 1024, sms, 0) == 256     # 20 x 4 tiles: doubling would spill into a second wave
    assert plan.gemm_bn(1024, 2048, sms, 0) == 128
    assert plan.gemm_bn(12288, 2048, sms, 128) == 128
