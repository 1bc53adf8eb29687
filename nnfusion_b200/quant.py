"""Packed low-bit weight formats of the dequantize-fused linear (host side, numpy).

The reference has no sub-byte element type (its list stops at ``u8``:
``src/nnfusion/common/type/element_type.hpp:41-55``), so packed uint4 tensors
travel through its runtime as ``uint8`` buffers and the layout below is this
library's own definition:

* weights  ``Wq``   uint4 ``[N, K]``      -> bytes ``[N, K/2]``; byte ``k/2`` of a row holds
  element ``k`` (even) in bits 0-3 and element ``k+1`` in bits 4-7;
* zero-points       uint4 ``[N, K/g]``    -> bytes ``[N, ceil(K/g / 2)]``, packed the same way
  along the group axis (an odd group count leaves the last high nibble zero);
* scales            fp16 (or fp32) ``[N, K/g]``, one per group of ``g`` consecutive K elements.

uint8 weights keep one byte per element, with uint8 zero-points ``[N, K/g]``.
"""
from __future__ import annotations

import numpy as np


def pack_u4(vals: np.ndarray) -> np.ndarray:
    """Pack uint4 values (one per uint8, last axis) two per byte, low nibble first."""
    vals = np.ascontiguousarray(vals, dtype=np.uint8)
    if vals.size and int(vals.max()) > 15:
        raise ValueError("pack_u4: values must be in 0..15")
    if vals.shape[-1] % 2:
        pad = np.zeros(vals.shape[:-1] + (1,), np.uint8)
        vals = np.concatenate([vals, pad], axis=-1)
    return np.ascontiguousarray(vals[..., 0::2] | (vals[..., 1::2] << 4))


def unpack_u4(packed: np.ndarray, n: int | None = None) -> np.ndarray:
    """Inverse of :func:`pack_u4`; ``n`` trims the padding nibble of an odd-length axis."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.uint8)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    return np.ascontiguousarray(out if n is None else out[..., :n])


def zp_row_bytes(K: int, group: int, bits: int) -> int:
    """Bytes per weight row of the zero-point tensor."""
    G = K // group
    return (G + 1) // 2 if bits == 4 else G
