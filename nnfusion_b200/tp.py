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


class PeerAllReduce:
    """Sum all-reduce of a small fp16 tensor through ``nnf_b200_allreduce_oneshot``: every rank's addend lives in
    memory that all ranks of the node have mapped (``torch.distributed._symmetric_memory``, i.e. ``cuMemMap`` of
    exported handles -- plumbing only), the kernel reads the peers' copies directly.

    ``addend(M)`` returns the view this rank must fill for the next call (two buffers alternate from call to call);
    ``__call__`` reduces what was written there into ``out``.
    """

    def __init__(self, max_elems: int, group, ctx=None):
        import ctypes

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib as L
        from .linear import default_context

        self.torch, self.ctypes = torch, ctypes
        dev = torch.device("cuda", torch.cuda.current_device())
        self.ctx = ctx or default_context(dev.index)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("the one-shot all-reduce serves up to 8 ranks of one node")
        self.max_elems = (max_elems + 7) // 8 * 8
        self.data_bytes = self.max_elems * 2
        flag_bytes = int(self.ctx.lib.nnf_b200_allreduce_flag_bytes(self.max_elems))
        self.flag_off = 2 * self.data_bytes
        total = (self.flag_off + flag_bytes + 255) // 256 * 256
        self.mem = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.mem.zero_()                       # flags start at zero on every rank ...
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.mem, group)
        dist.barrier(group)                    # ... before anybody's first flag store can arrive
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = 0
        vp = ctypes.c_void_p
        self._flags = (vp * self.world)(*[p + self.flag_off for p in self.ptrs])
        self._bufs = (vp * self.world)(*self.ptrs)

    def addend(self, shape):
        """The buffer this rank fills for the next call, viewed as fp16 ``shape``."""
        n = 1
        for d in shape:
            n *= d
        if n > self.max_elems or n % 8:
            raise ValueError("tensor too large for this all-reduce, or not a multiple of 8 elements")
        half = (self.epoch + 1) & 1
        return self.mem[half * self.data_bytes: half * self.data_bytes + 2 * n].view(self.torch.float16).view(shape)

    def __call__(self, out):
        """Call numbers are counted on the device, so a CUDA graph holding an even number of calls replays."""
        self.epoch += 1
        stream = self.torch.cuda.current_stream().cuda_stream
        rc = self.ctx.lib.nnf_b200_allreduce_oneshot(self.ctx.handle, stream, self.rank, self.world, self._bufs,
                                                     self._flags, out.numel(), self.data_bytes, out.data_ptr(), 0)
        self.ctx.check(rc)
        return out


class PeerLinear:
    """Row-parallel linear whose partial results are summed over the ranks inside the same launch
    (``nnf_b200_linear_allreduce``): y = sum_r x_r . dequant(W_r)^T.  ``weight`` is this rank's K shard."""

    def __init__(self, weight, group, max_rows: int = 16, ctx=None):
        import ctypes

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib as L
        from .linear import DequantDot, default_context

        self.torch, self.ctypes, self.L = torch, ctypes, L
        dev = weight.wq.device
        self.ctx = ctx or default_context(dev.index or 0)
        self.node = DequantDot(weight, ctx=self.ctx)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("the fused sum serves up to 8 ranks of one node")
        self.max_rows = max_rows
        self.half = (self.world * max_rows * weight.N * 4 + 255) // 256 * 256   # every sender's sums, per half
        d = self.node.desc(1, torch.float16)
        flag_bytes = int(self.ctx.lib.nnf_b200_linear_allreduce_flag_bytes(ctypes.byref(d)))
        self.flag_off = 2 * self.half
        total = (self.flag_off + flag_bytes + 255) // 256 * 256
        self.mem = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.mem.zero_()
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.mem, group)
        dist.barrier(group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        vp = ctypes.c_void_p
        self._bufs = (vp * self.world)(*ptrs)
        self._flags = (vp * self.world)(*[p + self.flag_off for p in ptrs])
        self._peers = L.Peers(self.rank, self.world, self._bufs, self._flags, self.half, 0)  # calls counted on device

    def __call__(self, x, out=None):
        torch, ctypes = self.torch, self.ctypes
        M = x.shape[0]
        if M > self.max_rows or x.dtype != torch.float16:
            raise ValueError("the fused sum serves fp16 activations of at most max_rows rows")
        if out is None:
            out = torch.empty((M, self.node.w.N), dtype=torch.float16, device=x.device)
        d = self.node.desc(M, x.dtype)
        ws = self.node.workspace(d)
        stream = torch.cuda.current_stream().cuda_stream
        rc = self.ctx.lib.nnf_b200_linear_allreduce(
            self.ctx.handle, stream, ctypes.byref(d), x.data_ptr(), ctypes.byref(self.node._abi_w), None,
            out.data_ptr(), ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            ctypes.byref(self._peers))
        self.ctx.check(rc)
        return out


class ShardedMLP:
    """This rank's part of y = down(SiLU(gate(x)) * up(x)), followed by the all-reduce.

    ``gate``/``up``/``down`` are device weights already sharded for this rank (``DeviceWeight``); ``group`` is the
    ``torch.distributed`` process group, or None for a single GPU.  ``gain`` enables the fused RMSNorm prologue of
    the gate/up linear (small-M kernel only).  ``reduce``: "nccl" (``torch.distributed.all_reduce``) or "peer" (the
    one-shot kernel over peer memory, fp16 outputs of at most ``peer_max_rows`` rows) or "fused" (the down linear
    sums over the ranks inside its own launch, same limits).
    """

    def __init__(self, gate, up, down, group=None, gain=None, eps: float = 1e-6, reduce: str = "nccl",
                 peer_max_rows: int = 16, peer: "Optional[PeerAllReduce]" = None):
        import torch

        from .linear import DequantDot

        self.torch = torch
        self.group = group
        self.gate_up = DequantDot(gate, up, gain=gain, eps=eps)
        self.down = DequantDot(down)
        self.hidden = down.N
        self._h = {}
        self._y = {}
        if reduce not in ("nccl", "peer", "fused"):
            raise ValueError("reduce must be 'nccl', 'peer' or 'fused'")
        self.fused = PeerLinear(down, group, peer_max_rows) if (reduce == "fused" and group is not None) else None
        # (several layers may share one PeerAllReduce: calls are ordered on the stream)
        self.peer = peer if peer is not None else (
            PeerAllReduce(peer_max_rows * down.N, group) if (reduce == "peer" and group is not None) else None)
        self.peer_max_rows = peer_max_rows

    def buffers(self, M: int, dtype, device):
        key = (M, dtype)
        if key not in self._h:
            self._h[key] = self.torch.empty((M, self.gate_up.w.N), dtype=dtype, device=device)
            self._y[key] = self.torch.empty((M, self.hidden), dtype=dtype, device=device)
        return self._h[key], self._y[key]

    def __call__(self, x):
        h, y = self.buffers(x.shape[0], x.dtype, x.device)
        self.gate_up(x, out=h)      # [M, inter / world]: SiLU(gate) * up, local
        if self.fused is not None and x.shape[0] <= self.peer_max_rows and x.dtype == self.torch.float16:
            return self.fused(h, out=y)  # partial sums exchanged and added inside the launch
        if self.peer is not None and x.shape[0] <= self.peer_max_rows and x.dtype == self.torch.float16:
            part = self.peer.addend((x.shape[0], self.hidden))
            self.down(h, out=part)  # partial sum over this rank's K shard, straight into peer-visible memory
            return self.peer(y)
        self.down(h, out=y)         # [M, hidden]: partial sum over this rank's K shard
        if self.group is not None:
            self.torch.distributed.all_reduce(y, group=self.group)
        return y

    @property
    def launches_per_step(self) -> int:
        return 3 if self.peer is not None else 2
