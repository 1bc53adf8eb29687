"""One LLaMA-style decoder layer at decode time (one token), built from the fused nodes of this package:

    x -> [RMSNorm -> q,k,v linears] -> [rotary, cache append, attention] -> [o linear + x]
      -> [RMSNorm -> SiLU(gate) * up] -> [down linear + residual]

Five launches where the reference's generated runtime runs some forty (element-wise dequantisation and cuBLAS Dot
per linear, the RMSNorm reduce / element-wise chain, the rotary element-wise kernels, two BatchMatMul and a Softmax;
see ``src/nnfusion/engine/pass/codegen/cuda_codegen_pass.cpp:248-430`` for how one kernel call per node is emitted).
PyTorch owns device memory and the stream; all arithmetic is in ``libnnf_b200.so``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .attention import DecodeAttention
from .linear import Context, DequantDot, DeviceWeight


class DecoderLayer:
    def __init__(self, q: DeviceWeight, k: DeviceWeight, v: DeviceWeight, o: DeviceWeight, gate: DeviceWeight,
                 up: DeviceWeight, down: DeviceWeight, attn_gain: torch.Tensor, mlp_gain: torch.Tensor, *,
                 heads: int, kv_heads: int, capacity: int, eps: float = 1e-6, rotary_base: float = 10000.0,
                 ctx: Optional[Context] = None):
        self.hidden = q.K
        self.head_dim = q.N // heads
        self.heads, self.kv_heads = heads, kv_heads
        if k.N != kv_heads * self.head_dim or v.N != k.N or o.K != q.N or down.N != self.hidden:
            raise ValueError("projection shapes do not describe one attention + MLP layer")
        dev = q.wq.device
        self.qkv = DequantDot(DeviceWeight.stack_rows([q, k, v]), gain=attn_gain, eps=eps, ctx=ctx)
        self.attn = DecodeAttention(heads, kv_heads, self.head_dim, capacity, dev, rotary_base=rotary_base, ctx=ctx)
        self.o = DequantDot(o, add=True, ctx=ctx)
        self.gate_up = DequantDot(gate, up, gain=mlp_gain, eps=eps, ctx=ctx)
        self.down = DequantDot(down, add=True, ctx=ctx)
        f16 = dict(dtype=torch.float16, device=dev)
        self._qkv = torch.empty((1, q.N + 2 * k.N), **f16)
        self._a = torch.empty((1, q.N), **f16)
        self._x1 = torch.empty((1, self.hidden), **f16)
        self._h = torch.empty((1, gate.N), **f16)
        self.launches = 5

    @property
    def weight_bytes(self) -> int:
        return sum(n.w.nbytes + (n.w2.nbytes if n.w2 is not None else 0)
                   for n in (self.qkv, self.o, self.gate_up, self.down))

    def __call__(self, x: torch.Tensor, position: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: fp16 [1, hidden], the residual stream; returns the layer's output [1, hidden]."""
        hd, kd = self.heads * self.head_dim, self.kv_heads * self.head_dim
        qkv = self.qkv(x, out=self._qkv)
        flat = qkv.view(-1)
        a = self.attn(flat[:hd], flat[hd:hd + kd], flat[hd + kd:], position, out=self._a)
        x1 = self.o(a, out=self._x1, addend=x)
        h = self.gate_up(x1, out=self._h)
        if out is None:
            out = torch.empty_like(x)
        return self.down(h, out=out, addend=x1)
