"""turq_qmatmul_static: the allocation-free variant of the integer-scheme matmul.

Some hosts cannot let a library allocate device memory while they run (their own pool owns
the GPU, or an allocation would stall their pipeline), so this entry keeps its activation
scratch in a fixed buffer inside the library. It must give exactly what the regular entry
gives, call after call, although every call reuses the same buffer. The file name sorts
last on purpose: a run that stops at the first failure has then covered everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _static_forward(lib, ctx, qt, x, bias=None):
    m = x.shape[0]
    y = torch.full((m, qt.shape()[0]), float("nan"), dtype=torch.float32, device=x.device)
    st = lib.turq_qmatmul_static(ctx.handle, qt._h, ctypes.c_void_p(x.data_ptr()), 0, m, ctypes.c_void_p(y.data_ptr()),
                                 ctypes.c_void_p(bias.data_ptr()) if bias is not None else None,
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, y


@pytest.mark.parametrize("dt", [oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K], ids=["Q8_0", "Q4_K", "Q5_K", "Q6_K"])
def test_static_entry_matches_regular_entry_on_consecutive_calls(dt):
    from tur_b200 import GgmlDType, Mode, QMatMul, QTensor, _lib, context
    lib = _lib.load()
    rng = np.random.default_rng(299792458 + dt)
    n, k = 304, 2048
    w = oracle.quantize(dt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    qt = QTensor.new(w, GgmlDType(dt), (n, k))
    ctx = context(qt.device())
    mm = QMatMul.from_arc(qt)
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    # two calls in a row on different inputs and row counts: the second must not see the first's planes
    for m, b in ((16, None), (3, bias), (16, bias)):
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
        st, y = _static_forward(lib, ctx, qt, x, b)
        assert st == 0, lib.turq_last_error(ctx.handle)
        want = mm.forward(x, bias=b, mode=Mode.INT8_ACT)
        assert torch.equal(y, want)                      # same kernels, same order: identical bits
        assert oracle.rel_fro(y.cpu().numpy(), oracle.qmatmul(dt, w, n, k, x.cpu().numpy())
                              + (b.cpu().numpy() if b is not None else 0)) < 2e-3


def test_static_entry_refuses_what_does_not_fit():
    from tur_b200 import GgmlDType, QTensor, _lib, context
    lib = _lib.load()
    n, k = 16, 8192
    w = oracle.quantize(oracle.Q4_K, np.zeros((n, k), np.float32))
    qt = QTensor.new(w, GgmlDType.Q4K, (n, k))
    ctx = context(qt.device())
    m = 1024                                          # 8 MiB of int8 activations alone
    x = torch.zeros((m, k), dtype=torch.float32, device="cuda")
    st, _ = _static_forward(lib, ctx, qt, x)
    assert st == 9 and b"static buffer" in lib.turq_last_error(ctx.handle)
    # 330 rows need 3.2 MB of planes: inside the 4 MiB array, but not beside its hand-over workspace
    st, _ = _static_forward(lib, ctx, qt, x[:330])
    assert st == 9 and b"hand-over workspace" in lib.turq_last_error(ctx.handle)
    st, y = _static_forward(lib, ctx, qt, x[:8])       # a refused call leaves the context usable
    assert st == 0 and torch.equal(y, torch.zeros_like(y))
    st, _ = _static_forward(lib, ctx, qt, x[:280])     # 2.7 MB of planes: fits
    assert st == 0


@pytest.mark.parametrize("n,k,m,why", [
    (9600, 4096, 2, "601 row-tiles on 296 CTA slots: row-tiles are cut between CTAs, partial sums and "
                    "ready flags go through the workspace at the tail of the static array"),
    (304, 1024, 1, "one row of 1024 values: the CTAs quantize the activations themselves, the array is only "
                   "used for its workspace"),
    (304, 4096, 9, "planes staged through the array and bulk-copied into shared memory"),
], ids=["cut_row_tiles", "in_kernel_quantization", "staged_planes"])
def test_static_entry_on_each_route_of_the_matmul(n, k, m, why):
    from tur_b200 import GgmlDType, Mode, QMatMul, QTensor, _lib, context
    lib = _lib.load()
    rng = np.random.default_rng(299792458 + n + m)
    w = oracle.quantize(oracle.Q4_K, (rng.standard_normal((min(n, 608), k)) * 0.02).astype(np.float32))
    w = np.ascontiguousarray(np.tile(w, (-(-n // w.shape[0]), 1))[:n])
    qt = QTensor.new(w, GgmlDType.Q4K, (n, k))
    ctx = context(qt.device())
    mm = QMatMul.from_arc(qt)
    for seed in (1, 2):                                # two calls in a row, different inputs
        x = torch.from_numpy(np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)).cuda()
        st, y = _static_forward(lib, ctx, qt, x)
        assert st == 0, lib.turq_last_error(ctx.handle)
        assert torch.equal(y, mm.forward(x, mode=Mode.INT8_ACT)), why
    ctx.poll_status()
