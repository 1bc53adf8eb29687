"""Python front door: run the quantised linears of a PyTorch module through this library.

The reference's front door traces a ``torch.nn.Module`` to ONNX, compiles it and swaps the module's ``forward`` for
the compiled runtime (``nnfusion.jit``: ``src/python/nnfusion/jit.py``; ``Session`` / ``Executor``:
``src/python/nnfusion/session.py``, ``src/python/nnfusion/executor.py:70-243``).  Its compiler cannot be built in
this environment, so its place is taken by the two ends of it that this package has: ``export_onnx`` writes a
``QuantLinear`` module as the ONNX graph an exporter would produce for it (Cast -> Sub -> Mul -> Gemm,
``onnx_writer.py``), ``compile_onnx`` reads such a file, folds the pattern the way the plugin's fold pass does and
returns the module bound to one ``nnf_b200_linear`` node.  ``jit`` wraps a module the way the reference's decorator
does (same call signature, torch tensors in and out, raw device pointers below), optionally sending every
``QuantLinear`` through that file stage.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import onnx_writer, synth
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


def export_onnx(m: QuantLinear, path: str, M: int, dtype: torch.dtype = torch.float16) -> None:
    """Writes ``m`` as the un-fused ONNX graph Y[M,N] = X[M,K] . ((Cast(Wq) - Cast(zp)) * scale)^T (+ bias)."""
    host = synth.QuantLinear.from_packed(m.out_features, m.in_features, m.bits, m.group_size,
                                         m.wq.cpu().numpy(), m.scale.cpu().numpy(), m.zp.cpu().numpy())
    np_dtype = np.float16 if dtype == torch.float16 else np.float32
    bias = m.bias.detach().cpu().numpy() if m.bias is not None else None
    onnx_writer.write_dequant_linear(path, host, M, np_dtype, bias)


def compile_onnx(path: str, bits: int = 8, device: str = "cuda") -> QuantLinear:
    """Reads an ONNX file holding the dequantised-linear pattern, folds it into one node and returns the module that
    runs it on ``device``.  ``bits`` = 4 packs the weights two per byte again (the file holds one byte per element)."""
    w, bias, _ = onnx_writer.fold_dequant_linear(onnx_writer.read_model(path), bits)
    return QuantLinear.from_host(w, None if bias is None else bias.astype(np.float32)).to(device)


def jit(module: torch.nn.Module, onnx_dir: Optional[str] = None) -> torch.nn.Module:
    """Prepare ``module`` for inference through this library: binds every ``QuantLinear`` inside it to its fused
    node (so the first call does not pay for it) and switches gradients off.  Returns the module, callable as
    before -- the reference's ``nnfusion.jit`` keeps the same contract.  With ``onnx_dir`` every ``QuantLinear`` is
    first exported to ``<onnx_dir>/<name>.onnx`` and replaced by what ``compile_onnx`` makes of that file, the way
    the reference goes through a file between tracing and compiling."""
    import os
    module.eval()
    for p in module.parameters():
        p.requires_grad_(False)
    if onnx_dir is not None:
        os.makedirs(onnx_dir, exist_ok=True)
        for name, m in list(module.named_modules()):
            if isinstance(m, QuantLinear) and name:
                path = os.path.join(onnx_dir, name.replace(".", "_") + ".onnx")
                dtype = torch.float16 if m.scale.dtype == torch.float16 else torch.float32
                export_onnx(m, path, 1, dtype)
                compiled = compile_onnx(path, m.bits, str(m.wq.device))
                parent = module
                *head, leaf = name.split(".")
                for part in head:
                    parent = getattr(parent, part)
                setattr(parent, leaf, compiled)
    for m in module.modules():
        if isinstance(m, QuantLinear) and m.wq.is_cuda:
            m.node()
    return module
