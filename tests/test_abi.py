"""CPU-side checks of the boundary: the library builds, loads, and exports exactly what the header declares."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import build, quant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build_library()
    return L.load()


def test_header_and_exports_agree(lib):
    hdr = open(os.path.join(ROOT, "include", "nnf_b200.h")).read()
    declared = sorted(set(re.findall(r"NNF_B200_API[^;]*?\b(nnf_b200_\w+)\s*\(", hdr)))
    assert declared == sorted(L.EXPORTS)
    out = subprocess.run(["nm", "-D", "--defined-only", L.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted(s for s in re.findall(r"\b(nnf_b200_\w+)\b", out))
    assert exported == declared            # nothing missing, nothing extra
    for name in declared:
        assert hasattr(lib, name)


def test_desc_layout_matches_header():
    assert ctypes.sizeof(L.LinearDesc) == 16 * 4
    assert ctypes.sizeof(L.QWeight) == 3 * ctypes.sizeof(ctypes.c_void_p)


def test_strerror(lib):
    assert lib.nnf_b200_strerror(L.OK) == b"ok"
    assert b"workspace" in lib.nnf_b200_strerror(L.EWORKSPACE)
    assert lib.nnf_b200_strerror(99) == b"unknown status"


def test_null_context_is_rejected(lib):
    assert lib.nnf_b200_linear(None, None, None, None, None, None, None, None, None, None, 0) == L.EINVAL
    assert lib.nnf_b200_last_error(None) == b""
    assert lib.nnf_b200_sm_count(None) == 0
    assert lib.nnf_b200_init(0, None) == L.EINVAL


def test_pack_u4_host_helper(lib):
    rng = np.random.default_rng(0)
    v = rng.integers(0, 16, size=(7, 33), dtype=np.uint8)
    out = np.zeros((7, 17), np.uint8)
    rc = lib.nnf_b200_pack_u4(v.tobytes(), 7, 33, out.ctypes.data_as(ctypes.c_char_p))
    assert rc == L.OK
    np.testing.assert_array_equal(out, quant.pack_u4(v))
    np.testing.assert_array_equal(quant.unpack_u4(out, 33), v)
    bad = v.copy()
    bad[0, 0] = 16
    assert lib.nnf_b200_pack_u4(bad.tobytes(), 7, 33, out.ctypes.data_as(ctypes.c_char_p)) == L.EINVAL
