"""Tensor-parallel SwiGLU MLP over the dequantize-fused linears: gate and up split by output row (column-parallel),
down split along K (row-parallel), one NCCL all-reduce of the [M, hidden] output at the shard boundary.

The reference's only collective is the data-parallel gradient all-reduce behind ``cuda::SuperScalerAllReduce``
(``src/nnfusion/core/kernels/cuda_gpu/kernels/allreduce.cpp:18-98``; NCCL call in
``src/tools/nnfusion/templates/super_scaler/super_scaler.cu:244-277``).  Here the same primitive (sum all-reduce on
the compute stream) closes a sharded layer instead.  One process per GPU, ``torch.distributed`` for the plumbing.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

from .synth import QuantLinear


def shard_rows_of_w(w: QuantLinear, rank: int, world: int) -> QuantLinear:
    """Column-parallel shard: output rows [rank * N/world, (rank+1) * N/world) of W[N, K] with their parameters."""
    if w.N % world:
        raise ValueError(f"N={w.N} is not divisible by {world} ranks")
    n = w.N // world
    sl = slice(rank * n, (rank + 1) * n)
    return QuantLinear(n, w.K, w.bits, w.group, np.ascontiguousarray(w.q[sl]), np.ascontiguousarray(w.scale[sl]),
                       np.ascontiguousarray(w.zp[sl]))


def shard_k_of_w(w: QuantLinear, rank: int, world: int) -> QuantLinear:
    """Row-parallel shard: K columns [rank * K/world, ...) of W[N, K]; shard boundaries fall on group boundaries."""
    if w.K % world or (w.K // world) % w.group:
        raise ValueError(f"K={w.K} cannot be split into {world} shards of whole groups of {w.group}")
    k = w.K // world
    g = k // w.group
    return QuantLinear(w.N, k, w.bits, w.group, np.ascontiguousarray(w.q[:, rank * k:(rank + 1) * k]),
                       np.ascontiguousarray(w.scale[:, rank * g:(rank + 1) * g]),
                       np.ascontiguousarray(w.zp[:, rank * g:(rank + 1) * g]))


def mlp_shapes(hidden: int, inter: int, world: int) -> Tuple[Tuple[int, int], Tuple[int, int]]:
    """Per-rank (N, K) of the gate/up shard and of the down shard."""
    if inter % world or (inter // world) % 128:
        raise ValueError(f"intermediate size {inter} cannot be sharded over {world} ranks in whole groups of 128")
    return (inter // world, hidden), (hidden, inter // world)


class ShardedMLP:
    """This rank's part of y = down(SiLU(gate(x)) * up(x)), followed by the all-reduce.

    ``gate``/``up``/``down`` are device weights already sharded for this rank (``DeviceWeight``); ``group`` is the
    ``torch.distributed`` process group, or None for a single GPU.  ``gain`` enables the fused RMSNorm prologue of
    the gate/up linear (small-M kernel only).
    """

    def __init__(self, gate, up, down, group=None, gain=None, eps: float = 1e-6):
        import torch

        from .linear import DequantDot

        self.torch = torch
        self.group = group
        self.gate_up = DequantDot(gate, up, gain=gain, eps=eps)
        self.down = DequantDot(down)
        self.hidden = down.N
        self._h = {}
        self._y = {}

    def buffers(self, M: int, dtype, device):
        key = (M, dtype)
        if key not in self._h:
            self._h[key] = self.torch.empty((M, self.gate_up.w.N), dtype=dtype, device=device)
            self._y[key] = self.torch.empty((M, self.hidden), dtype=dtype, device=device)
        return self._h[key], self._y[key]

    def __call__(self, x):
        h, y = self.buffers(x.shape[0], x.dtype, x.device)
        self.gate_up(x, out=h)      # [M, inter / world]: SiLU(gate) * up, local
        self.down(h, out=y)         # [M, hidden]: partial sum over this rank's K shard
        if self.group is not None:
            self.torch.distributed.all_reduce(y, group=self.group)
        return y

    @property
    def launches_per_step(self) -> int:
        return 2
