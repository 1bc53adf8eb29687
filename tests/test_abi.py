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
    # a launch with fewer units of work than SMs uses fewer CTAs, hence fewer slots; up to 64 batch rows the tile
    # (and with it a slot) is 64 rows wide instead of 256
    assert need(32, 128, 256) == 256 + 2 * 1 * 128 * 64 * 4
    assert need(65, 128, 256) == 256 + 2 * 1 * 128 * 256 * 4
    # small M: split-K scratch only
    assert need(1, 11008, 4096) < 1 << 20


def _plan(lib, M, N, K, bits=4, group=128, x=L.F16, scale=L.F16, epilogue=0, split_k=0, prologue=0):
    d = L.LinearDesc(M=M, N=N, K=K, w_bits=bits, group_size=group, x_dtype=x, y_dtype=x, scale_dtype=scale,
                     prologue=prologue, epilogue=epilogue, split_k=split_k)
    out = (ctypes.c_int32 * 8)()
    assert lib.nnf_b200_linear_plan(None, ctypes.byref(d), ctypes.byref(out)) == L.OK
    return dict(kernel=out[0], warps=out[1], splits=out[2], ctas=out[4], smem=out[5], batch=out[6],
                cluster=bool(out[7] & 1), l1_lines=bool(out[7] & 2), own_columns=bool(out[7] & 4),
                one_batch=bool(out[7] & 8))


def test_small_m_launch_shapes_without_a_device(lib):
    """The small-M planner's choices for the shapes whose timings the design notes quote (no context: a 148-SM
    device is assumed): how K is cut, which cuts may meet in a cluster's shared memory, which launches take L1
    lines for their weight loads, and how many tiles lie between two meetings of a CTA's warps."""
    silu = L.EPILOGUE_SILU_MUL
    # 7B decode: K = 4096 is 16 slices of 128 bytes, one CTA covers it; every tile of a CTA in one batch
    p = _plan(lib, 1, 11008, 4096)
    assert (p["kernel"], p["splits"], p["warps"], p["ctas"]) == (L.KERNEL_GEMV, 1, 16, 148)
    assert not p["cluster"] and not p["l1_lines"] and p["one_batch"] and p["batch"] == 5
    # K = 8192 has to be cut: in halves, which ask for clusters of two
    for N in (8192, 10240, 28672):
        p = _plan(lib, 1, N, 8192)
        assert p["splits"] == 2 and p["cluster"] and p["own_columns"] and not p["l1_lines"], (N, p)
    # two weight sets: halves as well (a three-way cut rates a little better on SM load alone), L1 lines only
    # when the pair is larger than L2
    p = _plan(lib, 1, 7168, 8192, epilogue=silu)
    assert p["splits"] == 2 and p["cluster"] and not p["l1_lines"]
    p = _plan(lib, 1, 28672, 8192, epilogue=silu)
    assert p["splits"] == 2 and p["cluster"] and p["l1_lines"] and p["one_batch"] and p["batch"] == 25
    # 70B down projection: K cut 7 ways (no cluster wish beyond what fits is decided at launch), L1 lines, one batch
    p = _plan(lib, 1, 8192, 28672)
    assert p["splits"] == 7 and p["l1_lines"] and p["own_columns"] and p["one_batch"] and p["batch"] == 25
    # 7B down projection: 43 slices, four ways, no L1 lines
    p = _plan(lib, 1, 4096, 11008)
    assert p["splits"] == 4 and not p["l1_lines"]
    # configuration 1: uint8 rows of 4096 bytes are 32 slices: halves, cluster
    p = _plan(lib, 16, 4096, 4096, bits=8, group=4096, x=L.F32, scale=L.F32)
    assert p["splits"] == 2 and p["cluster"]


@pytest.mark.parametrize("M", [1, 3, 8, 16])
@pytest.mark.parametrize("bits,group", [(4, 128), (8, 128), (8, 0)])
def test_small_m_plans_stay_inside_the_device(lib, M, bits, group):
    """Over a sweep of shapes: shared memory within the 227 KB a CTA may have, at most 16 warps, at most 32 tiles per
    batch, no more CTAs than four per SM, and a forced split honoured."""
    for N in (16, 160, 1024, 4096, 11008, 28672, 128256):
        for K in (256, 1024, 3584, 4096, 5120, 8192, 11008, 14336, 28672):
            g = group if group else K
            if K % g or (bits == 4 and K % 256) or K % 128:
                continue
            p = _plan(lib, M, N, K, bits=bits, group=g)
            if p["kernel"] != L.KERNEL_GEMV:
                continue
            assert 1 <= p["warps"] <= 16 and p["smem"] <= 227 * 1024, (N, K, p)
            assert 1 <= p["batch"] <= 32 and 1 <= p["ctas"] <= 4 * 148, (N, K, p)
            assert not p["cluster"] or 2 <= p["splits"] <= 8, (N, K, p)
