"""Python front door: run the quantised linears of a PyTorch module through this library.

The reference's front door traces a ``torch.nn.Module`` to ONNX, compiles it and swaps the module's ``forward`` for
the compiled runtime (``nnfusion.jit``: ``src/python/nnfusion/jit.py``; ``Session`` / ``Executor``:
``src/python/nnfusion/session.py``, ``src/python/nnfusion/executor.py:70-243``).  Its compiler cannot be built in
this environment, so the graph stage is skipped here: ``QuantLinear`` modules -- the Cast / Sub / Mul / Gemm pattern
of a dequantised linear, held packed -- are bound directly to ``nnf_b200_linear`` nodes, and ``jit`` wraps a module
the way the reference's decorator does (same call signature, torch tensors in and out, raw device pointers below).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import synth
from .linear import DequantDot, DeviceWeight


class QuantLinear(torch.nn.Module):
    """y = x . dequant(Wq)^T (+ bias): packed uint4 / uint8 weights with group-wise fp16 / fp32 scales and zero-points
    as buffers, so that ``state_dict`` / ``.to(device)`` carry them like any other parameter."""

    def __init__(self, in_features: int, out_features: int, bits: int = 4, group_size: int = 128,
                 bias: bool = False, scale_dtype: torch.dtype = torch.float16):
        super().__init__()
        if in_features % group_size:
            raise ValueError("in_features must be a multiple of group_size")
        G = in_features // group_size
        self.in_features, self.out_features, self.bits, self.group_size = in_features, out_features, bits, group_size
        self.register_buffer("wq", torch.zeros((out_features, in_features // 2 if bits == 4 else in_features),
                                               dtype=torch.uint8))
        self.register_buffer("scale", torch.ones((out_features, G), dtype=scale_dtype))
        self.register_buffer("zp", torch.zeros((out_features, (G + 1) // 2 if bits == 4 else G), dtype=torch.uint8))
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=torch.float32)) if bias else None
        self._node: Optional[DequantDot] = None

    @staticmethod
    def from_host(w: synth.QuantLinear, bias: Optional[np.ndarray] = None) -> "QuantLinear":
        m = QuantLinear(w.K, w.N, w.bits, w.group, bias is not None,
                        torch.float16 if w.scale.dtype == np.float16 else torch.float32)
        m.wq.copy_(torch.from_numpy(np.ascontiguousarray(w.wq)))
        m.scale.copy_(torch.from_numpy(np.ascontiguousarray(w.scale)))
        m.zp.copy_(torch.from_numpy(np.ascontiguousarray(w.zpq)))
        if bias is not None:
            with torch.no_grad():
                m.bias.copy_(torch.from_numpy(np.ascontiguousarray(bias, np.float32)))
        return m

    def dequantized(self) -> torch.Tensor:
        """fp32 [out, in]: what the reference's Convert -> Subtract -> Multiply chain would materialise (plain
        PyTorch, for tests and for exporting the un-fused graph)."""
        if self.bits == 4:
            q = torch.stack([self.wq & 0xF, self.wq >> 4], dim=-1).reshape(self.out_features, -1)
            z = torch.stack([self.zp & 0xF, self.zp >> 4], dim=-1).reshape(self.out_features, -1)
            z = z[:, : self.in_features // self.group_size]
        else:
            q, z = self.wq, self.zp
        q = q.to(torch.float32).reshape(self.out_features, -1, self.group_size)
        w = (q - z.to(torch.float32)[..., None]) * self.scale.to(torch.float32)[..., None]
        return w.reshape(self.out_features, self.in_features)

    def node(self) -> DequantDot:
        if self._node is None or self._node.w.wq.data_ptr() != self.wq.data_ptr():
            if not self.wq.is_cuda:
                raise RuntimeError("nnfusion_b200 runs on CUDA devices only: move the module to a GPU first")
            dw = DeviceWeight(self.out_features, self.in_features, self.bits, self.group_size, self.wq, self.scale,
                              self.zp)
            self._node = DequantDot(dw, bias=self.bias.data if self.bias is not None else None)
        return self._node

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = self.node()(x.reshape(-1, self.in_features).contiguous())
        return y.reshape(*lead, self.out_features)


def jit(module: torch.nn.Module) -> torch.nn.Module:
    """Prepare ``module`` for inference through this library: binds every ``QuantLinear`` inside it to its fused
    node (so the first call does not pay for it) and switches gradients off.  Returns the module, callable as
    before -- the reference's ``nnfusion.jit`` keeps the same contract."""
    module.eval()
    for p in module.parameters():
        p.requires_grad_(False)
    for m in module.modules():
        if isinstance(m, QuantLinear) and m.wq.is_cuda:
            m.node()
    return module
