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


def test_workspace_sizes_without_a_device(lib):
    """Sizing at code-generation time (no context: a 148-SM device is assumed).  Large M: the tiles' arrival counters,
    two fp32 tile slots per persistent CTA, and the fp16 copy of the activations when there is a pre-pass."""
    def need(M, N, K, x=L.F16, prologue=0):
        d = L.LinearDesc(M=M, N=N, K=K, w_bits=4, group_size=128, x_dtype=x, y_dtype=x, scale_dtype=L.F16,
                         prologue=prologue)
        return int(lib.nnf_b200_linear_workspace_bytes(None, ctypes.byref(d)))
    slots = 2 * 148 * 128 * 256 * 4
    tiles = 16 * 86                                  # 4096 / 256 batch tiles x 11008 / 128 weight-row tiles
    plain = need(4096, 11008, 4096)
    assert plain == (tiles * 4 + 255) // 256 * 256 + slots
    assert need(4096, 11008, 4096, x=L.F32) == plain + 4096 * 4096 * 2
    assert need(4096, 11008, 4096, prologue=L.PROLOGUE_RMSNORM) == plain + 4096 * 4096 * 2
    # a launch with fewer units of work than SMs uses fewer CTAs, hence fewer slots
    assert need(32, 128, 256) == 256 + 2 * 1 * 128 * 256 * 4
    # small M: split-K scratch only
    assert need(1, 11008, 4096) < 1 << 20
