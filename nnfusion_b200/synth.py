"""Seeded synthetic inputs with the shapes and value distributions of the benchmark graphs.

No dataset or checkpoint is involved: "LLaMA-7B/70B-shaped" means shapes only.  One
``numpy.random.Generator(PCG64(seed))`` stream is drawn in a fixed order per linear:
X ~ N(0,1) cast to its dtype, then Wq uniform integers, then scale ~ U(lo, hi), then
zero-points uniform integers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from .quant import pack_u4, unpack_u4


@dataclass
class QuantLinear:
    """One quantised weight matrix, unpacked (one uint8 per element / group) and packed."""
    N: int
    K: int
    bits: int
    group: int
    q: np.ndarray            # uint8 [N, K], values < 2**bits
    scale: np.ndarray        # fp16 or fp32 [N, K/group]
    zp: np.ndarray           # uint8 [N, K/group]

    @property
    def wq(self) -> np.ndarray:
        """Weight bytes as the kernels read them."""
        return pack_u4(self.q) if self.bits == 4 else self.q

    @property
    def zpq(self) -> np.ndarray:
        """Zero-point bytes as the kernels read them."""
        return pack_u4(self.zp) if self.bits == 4 else self.zp

    @staticmethod
    def from_packed(N: int, K: int, bits: int, group: int, wq: np.ndarray, scale: np.ndarray,
                    zpq: np.ndarray) -> "QuantLinear":
        """From the bytes the kernels read (the on-disk form) back to one value per element / group."""
        G = K // group
        if bits == 4:
            return QuantLinear(N, K, bits, group, unpack_u4(np.asarray(wq), K), np.asarray(scale),
                               unpack_u4(np.asarray(zpq), G))
        return QuantLinear(N, K, bits, group, np.asarray(wq), np.asarray(scale), np.asarray(zpq))


def make_weights(rng: np.random.Generator, N: int, K: int, bits: int, group: int,
                 scale_dtype=np.float16, scale_range=(0.002, 0.02),
                 zp_range: Optional[tuple] = None) -> QuantLinear:
    qmax = (1 << bits) - 1
    q = rng.integers(0, qmax + 1, size=(N, K), dtype=np.uint8)
    G = K // group
    scale = rng.uniform(scale_range[0], scale_range[1], size=(N, G)).astype(scale_dtype)
    lo, hi = zp_range if zp_range is not None else (0, qmax)
    zp = rng.integers(lo, hi + 1, size=(N, G), dtype=np.uint8)
    return QuantLinear(N, K, bits, group, q, scale, zp)


def make_x(rng: np.random.Generator, M: int, K: int, dtype) -> np.ndarray:
    return rng.standard_normal((M, K), dtype=np.float32).astype(dtype)


def config1(seed: int = 0, M: int = 16, N: int = 4096, K: int = 4096):
    """uint8 per-output-channel graph: X fp32 [M,K] ~N(0,1); W u8 [N,K] uniform 0..255;
    scale fp32 [N,1] ~U(0.001,0.01); zero-point u8 [N,1] uniform 120..136."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = make_x(rng, M, K, np.float32)
    w = make_weights(rng, N, K, 8, K, np.float32, (0.001, 0.01), (120, 136))
    return x, w


def u4g128(seed: int, M: int, N: int, K: int, x_dtype=np.float16):
    """uint4 group-128 linear: X fp16 ~N(0,1); W uniform 0..15; fp16 scale ~U(0.002,0.02);
    uint4 zero-points uniform 0..15."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = make_x(rng, M, K, x_dtype)
    w = make_weights(rng, N, K, 4, 128, np.float16, (0.002, 0.02))
    return x, w
