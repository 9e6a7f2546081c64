"""The C-ABI library: it loads, exports every symbol include/turq.h declares, its geometry
helpers agree with the oracle, and without a GPU it refuses to run instead of falling back."""
import ctypes
import os
import re

import pytest
import torch

import oracle
from tur_b200 import _lib
from tur_b200.build import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "turq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(turq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in turq.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table out of step with turq.h"


def test_version_and_status_strings(lib):
    assert lib.turq_version() == 100
    assert lib.turq_status_string(0) == b"ok"
    assert b"no CPU fallback" in lib.turq_status_string(8)


def test_geometry_matches_oracle(lib):
    for dt in (oracle.Q8_0, oracle.Q4_K, oracle.Q5_K, oracle.Q6_K, oracle.Q8_K, oracle.F32, oracle.F16, oracle.BF16):
        assert lib.turq_block_elems(dt) == oracle.block_elems(dt)
        assert lib.turq_block_bytes(dt) == oracle.block_bytes(dt)
    assert lib.turq_row_bytes(oracle.Q4_K, 4096) == 2304
    assert lib.turq_row_bytes(oracle.Q6_K, 2560) == 2100
    assert lib.turq_row_bytes(oracle.Q4_K, 100) == 0
    assert lib.turq_block_elems(99) == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_without_a_gpu_context_creation_fails_loudly(lib):
    h = ctypes.c_void_p()
    st = lib.turq_ctx_create(0, ctypes.byref(h))
    assert st == 8 and not h.value
    from tur_b200 import TurqError, context
    with pytest.raises(TurqError):
        context(0)


def test_null_arguments_are_rejected_not_dereferenced(lib):
    assert lib.turq_ctx_create(0, None) == 1
    assert lib.turq_ctx_destroy(None) == 1
    assert lib.turq_qtensor_free(None) == 1
    assert lib.turq_qtensor_info(None, None, None, None, None) == 1
    assert lib.turq_qmatmul(None, None, None, 0, 1, None, 0, None, None) == 1
    assert lib.turq_last_error(None) == b"null context"
