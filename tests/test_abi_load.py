"""CPU-side checks of the boundary: the shared library loads, exports every symbol the header
declares, and the pure-host entry points answer without a GPU."""
import os
import re

import pytest

from marlin_v100_b200 import _lib
from oracle import marlin_oracle as mo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from marlin_v100_b200 import build
        build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "marlin_b200.h")).read()
    declared = set(re.findall(r"\b(marlin_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_format_routing(lib):
    f = lib.marlin_b200_format_from_type_id
    assert f(mo.TYPE_U4B8, 0) == 0 and f(mo.TYPE_U4, 0) == 1
    assert f(mo.TYPE_U8B128, 0) == 2 and f(mo.TYPE_U8, 0) == 3
    assert f(mo.TYPE_FE4M3, 0) == 4
    assert f(mo.TYPE_FE2M1, 1) == 5 and f(mo.TYPE_FE2M1, 2) == 6
    assert f(mo.TYPE_FE2M1, 0) == -1 and f(12345, 0) == -1


def test_argument_errors_without_gpu(lib):
    # shape checks fire before any CUDA call
    rc = lib.marlin_b200_gptq_repack(None, None, None, 100, 64, 4, None)
    assert rc == -1 and b"size_k = 100 is not divisible" in lib.marlin_b200_last_error()
    rc = lib.marlin_b200_awq_repack(None, None, 64, 100, 4, None)
    assert rc == -1 and b"size_n = 100 is not divisible" in lib.marlin_b200_last_error()
    rc = lib.marlin_b200_gemm(None, None, None, None, None, None, None, 0, 0, 1, 100, 64, 64, 1, None, 0, None)
    assert rc == -1 and b"size_n % 64 == 0" in lib.marlin_b200_last_error()
    rc = lib.marlin_b200_gemm(None, None, None, None, None, None, None, 0, 0, 1, 64, 48, 48, 1, None, 0, None)
    assert rc == -1 and b"size_k % 32 == 0" in lib.marlin_b200_last_error()


def test_scalar_type_ids_match_oracle():
    from marlin_v100_b200 import scalar_types as st
    assert st.uint4.id == mo.TYPE_U4 and st.uint4b8.id == mo.TYPE_U4B8
    assert st.uint8.id == mo.TYPE_U8 and st.uint8b128.id == mo.TYPE_U8B128
    assert st.float4_e2m1f.id == mo.TYPE_FE2M1 and st.float8_e4m3fn.id == mo.TYPE_FE4M3
