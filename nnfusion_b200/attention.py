"""Host-side node for one decoding step of an attention layer (thin wrapper over ``nnf_b200_decode_attention``).

Mirrors the sub-graph the reference runs for it -- rotary embedding as element-wise kernels, ``BatchMatMul``
(``src/nnfusion/core/operators/generic_op/generic_op_define/BatchMatMul.cpp:6-50``), ``Softmax``, ``BatchMatMul`` --
as one node that owns the key/value caches the way the generated runtime owns persistent tensors.  PyTorch is used
for device memory and the current stream only.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib as L
from .linear import Context, default_context


class DecodeAttention:
    """Caches [kv_heads][capacity][head_dim] fp16; ``__call__`` appends the new token at ``position`` and returns
    the attention output [1, heads*head_dim]."""

    def __init__(self, heads: int, kv_heads: int, head_dim: int, capacity: int, device="cuda", *, rotary: bool = True,
                 rotary_base: float = 10000.0, softmax_scale: float = 0.0, splits: int = 0,
                 ctx: Optional[Context] = None):
        dev = torch.device(device)
        self.heads, self.kv_heads, self.head_dim, self.capacity = heads, kv_heads, head_dim, capacity
        self.rotary, self.rotary_base, self.softmax_scale, self.splits = rotary, rotary_base, softmax_scale, splits
        self.ctx = ctx or default_context(dev.index or 0)
        self.k_cache = torch.zeros((kv_heads, capacity, head_dim), dtype=torch.float16, device=dev)
        self.v_cache = torch.zeros((kv_heads, capacity, head_dim), dtype=torch.float16, device=dev)
        self._ws: dict = {}

    def desc(self, position: int) -> L.AttnDesc:
        d = L.AttnDesc()
        d.heads, d.kv_heads, d.head_dim, d.capacity = self.heads, self.kv_heads, self.head_dim, self.capacity
        d.position = position
        d.rotary = 1 if self.rotary else 0
        d.rotary_base, d.softmax_scale = self.rotary_base, self.softmax_scale
        d.splits = self.splits
        d.dtype = L.F16
        return d

    def workspace(self, d: L.AttnDesc) -> Optional[torch.Tensor]:
        n = int(self.ctx.lib.nnf_b200_decode_attention_workspace_bytes(self.ctx.handle, ctypes.byref(d)))
        if n == 0:
            return None
        ws = self._ws.get("ws")
        if ws is None or ws.numel() < n:
            # sized for the longest sequence the caches can hold, zeroed once
            full = self.desc(self.capacity - 1)
            cap = max(n, int(self.ctx.lib.nnf_b200_decode_attention_workspace_bytes(self.ctx.handle,
                                                                                   ctypes.byref(full))))
            raw = torch.empty(cap + 256, dtype=torch.uint8, device=self.k_cache.device)
            off = (-raw.data_ptr()) % 256
            ws = raw[off:off + cap]
            stream = torch.cuda.current_stream().cuda_stream
            self.ctx.check(self.ctx.lib.nnf_b200_workspace_reset(self.ctx.handle, stream, ws.data_ptr(), cap))
            self._ws["ws"] = ws
        return ws

    def __call__(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, position: int,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        hd, kd = self.heads * self.head_dim, self.kv_heads * self.head_dim
        for t, n in ((q, hd), (k_new, kd), (v_new, kd)):
            if t.dtype != torch.float16 or t.numel() != n or not t.is_contiguous():
                raise ValueError("q, k_new, v_new must be contiguous fp16 tensors of heads*head_dim elements")
        if out is None:
            out = torch.empty((1, hd), dtype=torch.float16, device=q.device)
        d = self.desc(position)
        ws = self.workspace(d)
        stream = torch.cuda.current_stream().cuda_stream
        rc = self.ctx.lib.nnf_b200_decode_attention(
            self.ctx.handle, stream, ctypes.byref(d), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
            self.k_cache.data_ptr(), self.v_cache.data_ptr(), out.data_ptr(),
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0)
        self.ctx.check(rc)
        return out
