"""CPU oracle for the dequantize-fused low-bit linear path (Python face).

TEST INFRASTRUCTURE ONLY.  Imported by ``tests/``, by the smoke check and by the
CPU-baseline legs of ``bench.py``; the shipped package never imports it.

Three implementations of the same arithmetic live here so that they can pin
one another:

* ``np_*``       numpy restatements (fp32 step by step), cheap to read;
* ``c_*``        ``liboracle.so`` built from ``oracle.c`` (plain C, OpenMP);
* ``ref_*``      ``_ref/libnnf_ref_mlas.so``: the reference's own vendored MLAS
                 SGEMM compiled from the reference checkout, behind the
                 elementwise kernels its CPU code generation emits.

Reference sources restated (paths relative to the reference project root):
Convert ``src/nnfusion/core/kernels/cpu/reference/kernels.cpp:711-719``;
Subtract/Multiply ``src/nnfusion/core/kernels/cpu/simd/elementwise.hpp:60-127``;
Broadcast ``src/nnfusion/core/operators/op_define/broadcast.cpp:71-117``;
Dot ``src/nnfusion/core/kernels/cpu/mlas/dot.cpp:89-100`` (MlasGemm NoTrans/Trans)
and the naive ``cpu_reference_dot`` ``.../reference/kernels.cpp:1532-1617``;
Sigmoid ``src/nnfusion/core/kernels/cuda_gpu/cuda_common_ops.hpp:96``.
Packed uint4, group-wise parameters, RMSNorm and SiLU*mul have no encoding in
the reference: parity for those is unpinned by the reference and rests on this
oracle.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libnnf_ref_mlas.so")

_lib = None
_ref = None


def build(ref: bool = True) -> None:
    """Compile ``liboracle.so`` and, when the reference checkout is present,
    ``_ref/libnnf_ref_mlas.so`` (recipe: the Makefile beside this file)."""
    target = "all" if ref else os.path.join(_HERE, "liboracle.so")
    subprocess.run(["make", "-s", "-C", _HERE, target], check=True)


def _ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


_F = ctypes.c_float
_U8 = ctypes.c_uint8
_U16 = ctypes.c_uint16
_SZ = ctypes.c_size_t
_PF = ctypes.POINTER(_F)
_PU8 = ctypes.POINTER(_U8)
_PU16 = ctypes.POINTER(_U16)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build(ref=False)
        L = ctypes.CDLL(_LIB_PATH)
        L.orc_convert_u8_f32.argtypes = [_PU8, _PF, _SZ]
        L.orc_convert_f16_f32.argtypes = [_PU16, _PF, _SZ]
        L.orc_convert_f32_f16.argtypes = [_PF, _PU16, _SZ]
        for name in ("orc_subtract_f32", "orc_multiply_f32", "orc_add_f32"):
            getattr(L, name).argtypes = [_PF, _PF, _PF, _SZ]
        L.orc_sigmoid_f32.argtypes = [_PF, _PF, _SZ]
        L.orc_broadcast_inner_f32.argtypes = [_PF, _PF, _SZ, _SZ]
        L.orc_unpack_u4.argtypes = [_PU8, _PU8, _SZ]
        L.orc_pack_u4.argtypes = [_PU8, _PU8, _SZ]
        L.orc_dot_naive.argtypes = [_PF, _PF, _PF, _SZ, _SZ, _SZ, ctypes.c_int]
        L.orc_sgemm_nt.argtypes = [_PF, _PF, _PF, _SZ, _SZ, _SZ]
        L.orc_dequant.argtypes = [_PU8, _PF, _PU8, _SZ, _SZ, _SZ, _PF]
        L.orc_rmsnorm_f32.argtypes = [_PF, _PF, _F, _PF, _SZ, _SZ]
        L.orc_silu_mul_f32.argtypes = [_PF, _PF, _PF, _SZ]
        L.orc_linear.argtypes = [_PF, _SZ, _SZ, _SZ, _SZ, _PU8, _PF, _PU8, _PU8, _PF, _PU8, _PF, _F,
                                 _PF, ctypes.c_int, _PF]
        L.orc_linear.restype = ctypes.c_int
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


def ref_lib() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        if not have_ref():
            raise FileNotFoundError(
                f"{_REF_PATH} is missing: build it with `make -C oracle` where the reference "
                "checkout is available")
        R = ctypes.CDLL(_REF_PATH)
        R.ref_mlas_sgemm.argtypes = [ctypes.c_int, ctypes.c_int, _SZ, _SZ, _SZ, _F, _PF, _SZ, _PF,
                                     _SZ, _F, _PF, _SZ]
        R.ref_num_threads.restype = ctypes.c_int
        R.ref_dequant_graph.argtypes = [_PU8, _PF, _PU8, _SZ, _SZ, _SZ, _PF, _PF]
        R.ref_linear_graph.argtypes = [_PF, _SZ, _SZ, _SZ, _SZ, _PU8, _PF, _PU8, _PF, _PF, _PF]
        _ref = R
    return _ref


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


# --------------------------------------------------------------------------- numpy restatement
def np_unpack_u4(packed: np.ndarray, n_elems: Optional[int] = None) -> np.ndarray:
    """Byte i holds element 2i in bits 0-3 and element 2i+1 in bits 4-7 (last axis)."""
    packed = _u8(packed)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.uint8)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    if n_elems is not None:
        out = out[..., :n_elems]
    return np.ascontiguousarray(out)


def np_pack_u4(vals: np.ndarray) -> np.ndarray:
    vals = _u8(vals)
    if vals.shape[-1] % 2:
        vals = np.concatenate([vals, np.zeros(vals.shape[:-1] + (1,), np.uint8)], axis=-1)
    return np.ascontiguousarray((vals[..., 0::2] & 0x0F) | ((vals[..., 1::2] & 0x0F) << 4))


def np_dequant(q: np.ndarray, scale: np.ndarray, zp: np.ndarray, group: int) -> np.ndarray:
    """Convert -> Subtract(Broadcast zp) -> Multiply(Broadcast scale), all fp32."""
    N, K = q.shape
    G = K // group
    wf = q.astype(np.float32).reshape(N, G, group)                       # Reshape + Convert
    zf = np.broadcast_to(zp.astype(np.float32).reshape(N, G, 1), wf.shape)  # Convert + Broadcast
    sf = np.broadcast_to(_f32(scale).reshape(N, G, 1), wf.shape)         # Broadcast
    t = wf - zf                                                          # Subtract
    return (t * sf).reshape(N, K)                                        # Multiply + Reshape


def np_rmsnorm(x: np.ndarray, gain: np.ndarray, eps: float) -> np.ndarray:
    x = _f32(x)
    ss = np.zeros(x.shape[0], np.float32)
    for k in range(x.shape[1]):  # sequential fp32 sum, as the C oracle
        ss = ss + x[:, k] * x[:, k]
    r = np.float32(1.0) / np.sqrt(ss / np.float32(x.shape[1]) + np.float32(eps))
    return x * r[:, None] * _f32(gain)[None, :]


def np_silu_mul(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    g = _f32(g)
    s = np.float32(1.0) / (np.float32(1.0) + np.exp(-g))
    return g * s * _f32(u)


def np_dot_f64(a: np.ndarray, b_nk: np.ndarray) -> np.ndarray:
    """High-precision second opinion: A[M,K] . B[N,K]^T accumulated in float64."""
    return a.astype(np.float64) @ b_nk.astype(np.float64).T


# --------------------------------------------------------------------------- C restatement
def c_dequant(q: np.ndarray, scale: np.ndarray, zp: np.ndarray, group: int) -> np.ndarray:
    q, scale, zp = _u8(q), _f32(scale), _u8(zp)
    N, K = q.shape
    out = np.empty((N, K), np.float32)
    lib().orc_dequant(_ptr(q, _U8), _ptr(scale, _F), _ptr(zp, _U8), N, K, group, _ptr(out, _F))
    return out


def c_dot(a: np.ndarray, b: np.ndarray, trans_b: bool, naive: bool = True) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    M, K = a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    out = np.empty((M, N), np.float32)
    if naive or not trans_b:
        lib().orc_dot_naive(_ptr(a, _F), _ptr(b, _F), _ptr(out, _F), M, N, K, int(trans_b))
    else:
        lib().orc_sgemm_nt(_ptr(a, _F), _ptr(b, _F), _ptr(out, _F), M, N, K)
    return out


def c_f16_to_f32(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, np.float16)
    out = np.empty(h.shape, np.float32)
    lib().orc_convert_f16_f32(_ptr(h.view(np.uint16), _U16), _ptr(out, _F), h.size)
    return out


def c_f32_to_f16(f: np.ndarray) -> np.ndarray:
    f = _f32(f)
    out = np.empty(f.shape, np.uint16)
    lib().orc_convert_f32_f16(_ptr(f, _F), _ptr(out, _U16), f.size)
    return out.view(np.float16)


def linear(x: np.ndarray, q: np.ndarray, scale: np.ndarray, zp: np.ndarray, group: int, *,
           q2: Optional[np.ndarray] = None, scale2: Optional[np.ndarray] = None,
           zp2: Optional[np.ndarray] = None, gain: Optional[np.ndarray] = None, eps: float = 1e-6,
           bias: Optional[np.ndarray] = None, out_dtype=None, naive_dot: bool = False) -> np.ndarray:
    """The whole linear graph on the C oracle.

    ``q``/``zp`` carry one uint8 per element / per group (uint4 already unpacked);
    ``scale``/``x``/``gain``/``bias`` may be fp16 or fp32 and are upcast on entry; the
    fp32 result is rounded once to ``out_dtype`` (default: dtype of ``x``)."""
    out_dtype = np.dtype(out_dtype or x.dtype)
    xf = _f32(x)
    M, K = xf.shape
    q = _u8(q)
    N = q.shape[0]
    assert q.shape == (N, K) and K % group == 0
    G = K // group
    sc = _f32(np.asarray(scale).reshape(N, G))
    z = _u8(np.asarray(zp).reshape(N, G))
    y = np.empty((M, N), np.float32)
    null_f = ctypes.cast(None, _PF)
    null_u8 = ctypes.cast(None, _PU8)
    keep = []

    def opt_f(a):
        if a is None:
            return null_f
        a = _f32(a)
        keep.append(a)
        return _ptr(a, _F)

    def opt_u8(a, shape=None):
        if a is None:
            return null_u8
        a = _u8(np.asarray(a).reshape(shape) if shape else a)
        keep.append(a)
        return _ptr(a, _U8)

    rc = lib().orc_linear(_ptr(xf, _F), M, N, K, group, _ptr(q, _U8), _ptr(sc, _F), _ptr(z, _U8),
                          opt_u8(q2), opt_f(None if scale2 is None else np.asarray(scale2).reshape(N, G)),
                          opt_u8(zp2, (N, G)), opt_f(gain), float(eps), opt_f(bias),
                          int(naive_dot), _ptr(y, _F))
    if rc != 0:
        raise MemoryError("orc_linear: scratch allocation failed")
    if out_dtype == np.float16:
        return c_f32_to_f16(y)
    return y


# --------------------------------------------------------------------------- compiled reference
def ref_sgemm(a: np.ndarray, b: np.ndarray, trans_a: bool = False, trans_b: bool = False,
              alpha: float = 1.0, beta: float = 0.0, c: Optional[np.ndarray] = None) -> np.ndarray:
    """MlasGemm from the reference's vendored MLAS (row-major, like the CPU code generation)."""
    a, b = _f32(a), _f32(b)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    out = np.zeros((M, N), np.float32) if c is None else _f32(c).copy()
    ref_lib().ref_mlas_sgemm(int(trans_a), int(trans_b), M, N, K, alpha, _ptr(a, _F), a.shape[1],
                             _ptr(b, _F), b.shape[1], beta, _ptr(out, _F), N)
    return out


class RefLinearGraph:
    """The reference CPU graph for one dequantised linear (Convert, Subtract, Multiply through
    restated elementwise kernels, Dot through the reference's MLAS), with its fp32 [N,K]
    intermediates allocated once like the generated runtime's memory pool."""

    def __init__(self, N: int, K: int):
        self.N, self.K = N, K
        self.wf = np.empty((N, K), np.float32)
        self.wdq = np.empty((N, K), np.float32)

    def __call__(self, x: np.ndarray, q: np.ndarray, scale: np.ndarray, zp: np.ndarray,
                 group: int) -> np.ndarray:
        x, q = _f32(x), _u8(q)
        M = x.shape[0]
        G = self.K // group
        sc = _f32(np.asarray(scale).reshape(self.N, G))
        z = _u8(np.asarray(zp).reshape(self.N, G))
        y = np.empty((M, self.N), np.float32)
        ref_lib().ref_linear_graph(_ptr(x, _F), M, self.N, self.K, group, _ptr(q, _U8), _ptr(sc, _F),
                                   _ptr(z, _U8), _ptr(self.wf, _F), _ptr(self.wdq, _F), _ptr(y, _F))
        return y

    def gemm_only(self, x: np.ndarray) -> np.ndarray:
        """Dot alone on the already dequantised weights (what runs when constants are folded)."""
        return ref_sgemm(x, self.wdq, trans_b=True)


def ref_threads() -> int:
    return int(ref_lib().ref_num_threads())


# --------------------------------------------------------------------------- comparison metric
def max_rel_err(y: np.ndarray, r: np.ndarray) -> float:
    """max|y - r| / max|r|: outputs are zero-mean, so element-wise relative error is unbounded
    near zero; the gated figure normalises by the largest reference magnitude."""
    y64, r64 = np.asarray(y, np.float64), np.asarray(r, np.float64)
    denom = float(np.max(np.abs(r64))) if r64.size else 0.0
    if denom == 0.0:
        return float(np.max(np.abs(y64 - r64))) if r64.size else 0.0
    return float(np.max(np.abs(y64 - r64)) / denom)
