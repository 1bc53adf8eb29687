"""CPU oracle for one decoding step of an attention layer (rotary embedding, cache append, q.K^T, softmax, P.V).

TEST INFRASTRUCTURE ONLY.  Imported by ``tests/``, by the smoke check and by the CPU-baseline legs of
``bench.py``; the shipped package never imports it.

Each function restates what the reference executes for that operator on its CPU path (paths relative to the
reference project root), in fp32 step by step:

* ``batch_matmul``  ``cpu::BatchMatMulMlas`` -- one ``MlasGemm`` per batch entry with the ``adj_x`` / ``adj_y``
  flags as transposes (``src/nnfusion/core/kernels/cpu/mlas/batch_matmul.cpp:9-119``; operator definition and shape
  rules ``src/nnfusion/core/operators/generic_op/generic_op_define/BatchMatMul.cpp:6-50``).  ``ref_batch_matmul``
  runs the reference's own compiled MLAS for every batch entry.
* ``softmax``       ``cpu_reference_softmax`` (``src/nnfusion/core/kernels/cpu/reference/kernels.cpp:1856-1885``):
  maximum over the axes, ``exp(x - max)``, sum, divide.
* ``rotate_half``   the element-wise graph a frontend emits for the rotary embedding: Slice, Negative, Concat,
  Multiply, Add (``src/nnfusion/core/kernels/cuda_gpu/cuda_common_ops.hpp:28-97`` for the element-wise formulas).
  The angle table itself (``position * base**(-2i/d)``) is computed by the caller of the reference, i.e. it is a
  model constant; here it is computed in float64 and rounded to fp32.

Pinned by the reference's own vectors where it has any: softmax of ones(2,3,5) is 0.2 everywhere
(``test/nnfusion/frontend/torchscript_import.cpp:160-190``); the matrix products against the compiled MLAS.  The
rotary convention, the cache layout [kv_heads][capacity][head_dim] and grouped queries have no encoding in the
reference: parity for those is unpinned by the reference and rests on this oracle.
"""
from __future__ import annotations

import numpy as np

from . import oracle as _o


def batch_matmul(a: np.ndarray, b: np.ndarray, adj_x: bool = False, adj_y: bool = False) -> np.ndarray:
    """``a``, ``b``: [..., r, c] with equal leading dimensions, fp32; float64 accumulation rounded once (the
    order-free answer that the K-blocked fp32 SGEMM is compared against with a tolerance)."""
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    if a.shape[:-2] != b.shape[:-2]:
        raise ValueError("leading dimensions must match (BatchMatMul.cpp:24-30)")
    x = np.swapaxes(a, -1, -2) if adj_x else a
    y = np.swapaxes(b, -1, -2) if adj_y else b
    if x.shape[-1] != y.shape[-2]:
        raise ValueError("contraction dimensions differ")
    return np.matmul(x.astype(np.float64), y.astype(np.float64)).astype(np.float32)


def ref_batch_matmul(a: np.ndarray, b: np.ndarray, adj_x: bool = False, adj_y: bool = False) -> np.ndarray:
    """The same through the reference's compiled MLAS, one SGEMM per batch entry as its CPU emitter does."""
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    lead = a.shape[:-2]
    a2 = a.reshape((-1,) + a.shape[-2:])
    b2 = b.reshape((-1,) + b.shape[-2:])
    outs = [_o.ref_sgemm(a2[i], b2[i], trans_a=adj_x, trans_b=adj_y) for i in range(a2.shape[0])]
    return np.stack(outs).reshape(lead + outs[0].shape)


def softmax(x: np.ndarray, axis: int = -1) -> np.ndarray:
    x = np.asarray(x, np.float32)
    m = np.max(x, axis=axis, keepdims=True)
    e = np.exp(x - m).astype(np.float32)
    s = np.sum(e, axis=axis, keepdims=True, dtype=np.float32)
    return (e / s).astype(np.float32)


def rotary_tables(position: int, head_dim: int, base: float = 10000.0):
    """cos / sin of position * base**(-2i/head_dim), i < head_dim/2, repeated over both halves; fp32."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    ang = position * base ** (-2.0 * i / head_dim)
    cos = np.concatenate([np.cos(ang), np.cos(ang)]).astype(np.float32)
    sin = np.concatenate([np.sin(ang), np.sin(ang)]).astype(np.float32)
    return cos, sin


def rotate_half(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x [..., head_dim] fp32 -> x*cos + concat(-x[half:], x[:half])*sin (Slice, Negative, Concat, Multiply, Add)."""
    x = np.asarray(x, np.float32)
    h = x.shape[-1] // 2
    rot = np.concatenate([-x[..., h:], x[..., :h]], axis=-1)
    return (x * cos + rot * sin).astype(np.float32)


def decode_attention(q: np.ndarray, k_new: np.ndarray, v_new: np.ndarray, k_cache: np.ndarray,
                     v_cache: np.ndarray, position: int, *, rotary: bool = True, base: float = 10000.0,
                     scale: float = 0.0, use_ref: bool = False):
    """One decoding step.  q [H,D], k_new / v_new [Hkv,D], caches [Hkv,capacity,D], all fp16.

    Returns (out fp16 [H,D], new key row fp16 [Hkv,D] as appended to the cache).  The caches are updated in
    place at row ``position``.  fp16 tensors are widened to fp32 on entry; the appended key is rounded to fp16
    (the cache's element type) and that rounded row is what the product sees; the output is rounded once.
    """
    H, D = q.shape
    Hkv = k_new.shape[0]
    qf = np.asarray(q, np.float16).astype(np.float32)
    kf = np.asarray(k_new, np.float16).astype(np.float32)
    if rotary:
        cos, sin = rotary_tables(position, D, base)
        qf = rotate_half(qf, cos, sin)
        kf = rotate_half(kf, cos, sin)
    k_row = kf.astype(np.float16)
    k_cache[:, position, :] = k_row
    v_cache[:, position, :] = np.asarray(v_new, np.float16)
    n = position + 1
    rep = H // Hkv
    K = np.repeat(k_cache[:, :n, :].astype(np.float32), rep, axis=0)  # [H, n, D]
    V = np.repeat(v_cache[:, :n, :].astype(np.float32), rep, axis=0)
    sc = np.float32(scale if scale > 0 else 1.0 / np.sqrt(D))
    bmm = ref_batch_matmul if use_ref else batch_matmul
    s = bmm(qf[:, None, :], K, adj_y=True) * sc                      # [H, 1, n]
    p = softmax(s, axis=-1)
    o = bmm(p, V)                                                     # [H, 1, D]
    return o[:, 0, :].astype(np.float16), k_row
