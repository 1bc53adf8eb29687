"""ctypes binding of ``libnnf_b200.so`` (declarations: ``include/nnf_b200.h``).

There is no fallback: if the library is missing or fails to load, importing callers get a
``RuntimeError`` that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libnnf_b200.so")

OK, EINVAL, ENOTSUP, ECUDA, EWORKSPACE, ETIMEDOUT, EALIGN = range(7)
F32, F16 = 0, 1
PROLOGUE_NONE, PROLOGUE_RMSNORM = 0, 1
EPILOGUE_NONE, EPILOGUE_BIAS, EPILOGUE_SILU_MUL, EPILOGUE_ADD = 0, 1, 2, 3
KERNEL_AUTO, KERNEL_GEMV, KERNEL_GEMM = 0, 1, 2
FLAG_EXACT_ZP = 1
STATIC_SCRATCH_BYTES = 4 * 1024 * 1024

# Every symbol include/nnf_b200.h declares.
EXPORTS = (
    "nnf_b200_init", "nnf_b200_free", "nnf_b200_strerror", "nnf_b200_last_error", "nnf_b200_sm_count",
    "nnf_b200_linear_workspace_bytes", "nnf_b200_workspace_reset", "nnf_b200_linear",
    "nnf_b200_launch_count", "nnf_b200_pack_u4", "nnf_b200_device_status", "nnf_b200_linear_plan",
    "nnf_b200_linear_static_scratch", "nnf_b200_static_scratch_status", "nnf_b200_decode_attention_workspace_bytes", "nnf_b200_decode_attention",
    "nnf_b200_allreduce_flag_bytes", "nnf_b200_allreduce_oneshot",
    "nnf_b200_linear_allreduce_flag_bytes", "nnf_b200_linear_allreduce",
)


class LinearDesc(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("w_bits", ctypes.c_int32), ("group_size", ctypes.c_int32),
        ("x_dtype", ctypes.c_int32), ("y_dtype", ctypes.c_int32), ("scale_dtype", ctypes.c_int32),
        ("prologue", ctypes.c_int32), ("epilogue", ctypes.c_int32), ("rms_eps", ctypes.c_float),
        ("kernel", ctypes.c_int32), ("split_k", ctypes.c_int32), ("flags", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 2),
    ]


class AttnDesc(ctypes.Structure):
    _fields_ = [
        ("heads", ctypes.c_int32), ("kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("capacity", ctypes.c_int32), ("position", ctypes.c_int32), ("rotary", ctypes.c_int32),
        ("rotary_base", ctypes.c_float), ("softmax_scale", ctypes.c_float),
        ("splits", ctypes.c_int32), ("dtype", ctypes.c_int32), ("reserved", ctypes.c_int32 * 4),
    ]


class Peers(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("bufs", ctypes.POINTER(ctypes.c_void_p)),
                ("flags", ctypes.POINTER(ctypes.c_void_p)), ("half_stride_bytes", ctypes.c_size_t),
                ("epoch", ctypes.c_uint32)]


class QWeight(ctypes.Structure):
    _fields_ = [("wq", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("zp", ctypes.c_void_p)]


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: build it with `python -m nnfusion_b200.build` "
            "(nvcc, sm_100a); there is no CPU or PyTorch fallback")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    L.nnf_b200_init.argtypes = [ctypes.c_int, ctypes.POINTER(vp)]
    L.nnf_b200_free.argtypes = [vp]
    L.nnf_b200_strerror.argtypes = [ctypes.c_int]
    L.nnf_b200_strerror.restype = ctypes.c_char_p
    L.nnf_b200_last_error.argtypes = [vp]
    L.nnf_b200_last_error.restype = ctypes.c_char_p
    L.nnf_b200_sm_count.argtypes = [vp]
    L.nnf_b200_linear_workspace_bytes.argtypes = [vp, ctypes.POINTER(LinearDesc)]
    L.nnf_b200_linear_workspace_bytes.restype = sz
    L.nnf_b200_workspace_reset.argtypes = [vp, vp, vp, sz]
    L.nnf_b200_linear.argtypes = [vp, vp, ctypes.POINTER(LinearDesc), vp, ctypes.POINTER(QWeight),
                                  ctypes.POINTER(QWeight), vp, vp, vp, vp, sz]
    L.nnf_b200_device_status.argtypes = [vp, vp]
    L.nnf_b200_linear_static_scratch.argtypes = [vp, ctypes.POINTER(LinearDesc), vp, ctypes.POINTER(QWeight),
                                                 ctypes.POINTER(QWeight), vp, vp, vp, ctypes.c_char_p, sz]
    L.nnf_b200_static_scratch_status.argtypes = [vp]
    L.nnf_b200_linear_plan.argtypes = [vp, ctypes.POINTER(LinearDesc), ctypes.POINTER(ctypes.c_int32 * 8)]
    L.nnf_b200_launch_count.argtypes = [vp, ctypes.c_int]
    L.nnf_b200_launch_count.restype = ctypes.c_uint64
    L.nnf_b200_pack_u4.argtypes = [ctypes.c_char_p, sz, sz, ctypes.c_char_p]
    L.nnf_b200_decode_attention_workspace_bytes.argtypes = [vp, ctypes.POINTER(AttnDesc)]
    L.nnf_b200_decode_attention_workspace_bytes.restype = sz
    L.nnf_b200_decode_attention.argtypes = [vp, vp, ctypes.POINTER(AttnDesc), vp, vp, vp, vp, vp, vp, vp, sz]
    L.nnf_b200_linear_allreduce_flag_bytes.argtypes = [ctypes.POINTER(LinearDesc)]
    L.nnf_b200_linear_allreduce_flag_bytes.restype = sz
    L.nnf_b200_linear_allreduce.argtypes = [vp, vp, ctypes.POINTER(LinearDesc), vp, ctypes.POINTER(QWeight), vp, vp,
                                            vp, sz, ctypes.POINTER(Peers)]
    L.nnf_b200_allreduce_flag_bytes.argtypes = [sz]
    L.nnf_b200_allreduce_flag_bytes.restype = sz
    L.nnf_b200_allreduce_oneshot.argtypes = [vp, vp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(vp),
                                             ctypes.POINTER(vp), sz, sz, vp, ctypes.c_uint32]
    _lib = L
    return L
