"""Host-side face of the fused dequantised linear, in the vocabulary of the reference's
operator interface: a ``DequantDot`` node holds the quantised ``Constant`` tensors of one Dot
and is executed by a kernel that receives raw device pointers on a stream, exactly like a
``CudaLibEmitter`` body in the generated ``kernel_entry``
(``src/nnfusion/core/kernels/cuda_gpu/cuda_emitter.hpp:190-199``).

PyTorch is used only to own device memory and the current stream.  All arithmetic runs in
``libnnf_b200.so``; there is no fallback.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib as L
from .synth import QuantLinear


class NNFB200Error(RuntimeError):
    def __init__(self, status: int, text: str, detail: str):
        super().__init__(f"nnf_b200: {text} (status {status}): {detail}")
        self.status = status


class Context:
    """One per device; wraps ``nnf_b200_init`` / ``nnf_b200_free``."""

    def __init__(self, device: int = 0):
        self.lib = L.load()
        self.handle = ctypes.c_void_p()
        self.device = device
        rc = self.lib.nnf_b200_init(device, ctypes.byref(self.handle))
        if rc != L.OK:
            raise NNFB200Error(rc, self.lib.nnf_b200_strerror(rc).decode(), "nnf_b200_init")

    def check(self, rc: int) -> None:
        if rc != L.OK:
            raise NNFB200Error(rc, self.lib.nnf_b200_strerror(rc).decode(),
                               self.lib.nnf_b200_last_error(self.handle).decode())

    @property
    def sm_count(self) -> int:
        return int(self.lib.nnf_b200_sm_count(self.handle))

    def device_status(self) -> None:
        """Raise if a bounded device-side wait gave up since the last query (synchronises)."""
        import torch
        self.check(self.lib.nnf_b200_device_status(self.handle, torch.cuda.current_stream().cuda_stream))

    def launch_count(self, reset: bool = False) -> int:
        return int(self.lib.nnf_b200_launch_count(self.handle, int(reset)))

    def close(self) -> None:
        if self.handle:
            self.lib.nnf_b200_free(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


_contexts: dict = {}


def default_context(device: int = 0) -> Context:
    if device not in _contexts:
        _contexts[device] = Context(device)
    return _contexts[device]


_DT = {torch.float32: L.F32, torch.float16: L.F16}


@dataclass
class DeviceWeight:
    """Quantised weight tensors resident in device memory, as the kernels read them."""
    N: int
    K: int
    bits: int
    group: int
    wq: torch.Tensor     # uint8 [N, K/2] (4-bit) or [N, K]
    scale: torch.Tensor  # fp16 / fp32 [N, K/group]
    zp: torch.Tensor     # uint8 packed like the weights along the group axis

    @staticmethod
    def from_host(w: QuantLinear, device: str = "cuda:0") -> "DeviceWeight":
        return DeviceWeight(w.N, w.K, w.bits, w.group,
                            torch.from_numpy(np.ascontiguousarray(w.wq)).to(device),
                            torch.from_numpy(np.ascontiguousarray(w.scale)).to(device),
                            torch.from_numpy(np.ascontiguousarray(w.zpq)).to(device))

    @staticmethod
    def stack_rows(parts: "list[DeviceWeight]") -> "DeviceWeight":
        """Weights that read the same activations, concatenated along N (a constant-folding-time Concat):
        q, k and v of an attention layer become one matrix and one launch."""
        first = parts[0]
        if any((p.K, p.bits, p.group, p.scale.dtype) != (first.K, first.bits, first.group, first.scale.dtype)
               for p in parts):
            raise ValueError("stacked weights must share K, bit width, group size and scale type")
        return DeviceWeight(sum(p.N for p in parts), first.K, first.bits, first.group,
                            torch.cat([p.wq for p in parts]).contiguous(),
                            torch.cat([p.scale for p in parts]).contiguous(),
                            torch.cat([p.zp for p in parts]).contiguous())

    def shard_rows(self, rank: int, world: int) -> "DeviceWeight":
        """Column-parallel shard on the device: output rows [rank * N/world, (rank+1) * N/world) with their parameters."""
        if self.N % world:
            raise ValueError(f"N={self.N} is not divisible by {world} ranks")
        n = self.N // world
        sl = slice(rank * n, (rank + 1) * n)
        return DeviceWeight(n, self.K, self.bits, self.group, self.wq[sl].contiguous(), self.scale[sl].contiguous(),
                            self.zp[sl].contiguous())

    def shard_k(self, rank: int, world: int) -> "DeviceWeight":
        """Row-parallel shard on the device: K columns [rank * K/world, ...); shards hold whole groups, and for 4-bit
        weights an even number of them (the packed zero-points split on a byte boundary)."""
        k = self.K // world
        g = k // self.group if self.group else 0
        if self.K % world or g * self.group != k or (self.bits == 4 and g % 2):
            raise ValueError(f"K={self.K} cannot be split into {world} shards of whole (pairs of) groups of {self.group}")
        per = 2 if self.bits == 4 else 1
        return DeviceWeight(self.N, k, self.bits, self.group,
                            self.wq[:, rank * k // per:(rank + 1) * k // per].contiguous(),
                            self.scale[:, rank * g:(rank + 1) * g].contiguous(),
                            self.zp[:, rank * g // per:(rank + 1) * g // per].contiguous())

    def abi(self) -> L.QWeight:
        return L.QWeight(self.wq.data_ptr(), self.scale.data_ptr(), self.zp.data_ptr())

    @property
    def nbytes(self) -> int:
        return self.wq.numel() + self.scale.numel() * self.scale.element_size() + self.zp.numel()


class DequantDot:
    """y = epilogue(prologue(x) . dequant(W)^T) for one quantised weight (or a gate/up pair).

    Mirrors the fused graph node that stands in for Convert -> Subtract -> Multiply -> Dot(transB)
    (``src/nnfusion/core/operators/op_define/dot.cpp:43-135``).  The workspace is allocated once
    per (node, M) and zeroed once, as the generated runtime plans temp tensors into its pool
    (``src/nnfusion/core/kernels/kernel_emitter.cpp:282-319``).
    """

    def __init__(self, weight: DeviceWeight, weight2: Optional[DeviceWeight] = None,
                 gain: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                 eps: float = 1e-6, y_dtype: Optional[torch.dtype] = None, kernel: int = L.KERNEL_AUTO,
                 split_k: int = 0, flags: int = 0, ctx: Optional[Context] = None, add: bool = False,
                 kernel_db=None, db_device: str = "B200"):
        self.w, self.w2, self.gain, self.bias = weight, weight2, gain, bias
        # measured launch choices (nnfusion_b200.kernel_db.KernelCacheManager); entries found there override the
        # built-in rule, like the reference's FetchBasedSelector overrides priorities
        self.kernel_db, self.db_device = kernel_db, db_device
        self.add = add  # y = x.W^T + addend, the addend ([M,N], y's dtype) being given at call time
        if add and (bias is not None or weight2 is not None):
            raise ValueError("the add epilogue excludes bias and the SiLU*mul epilogue")
        self.eps, self.y_dtype, self.kernel, self.split_k, self.flags = eps, y_dtype, kernel, split_k, flags
        self.ctx = ctx or default_context(weight.wq.device.index or 0)
        if weight2 is not None and (weight2.N, weight2.K, weight2.bits, weight2.group) != \
                (weight.N, weight.K, weight.bits, weight.group):
            raise ValueError("gate and up weights must share shape and format")
        if gain is not None and gain.dtype != torch.float32:
            raise ValueError("RMSNorm gain must be fp32")
        if bias is not None and bias.dtype != torch.float32:
            raise ValueError("bias must be fp32")
        self._ws: dict = {}
        self._abi_w = weight.abi()
        self._abi_w2 = weight2.abi() if weight2 is not None else None

    def desc(self, M: int, x_dtype: torch.dtype) -> L.LinearDesc:
        d = L.LinearDesc()
        d.M, d.N, d.K = M, self.w.N, self.w.K
        d.w_bits = self.w.bits
        d.group_size = self.w.group
        d.x_dtype = _DT[x_dtype]
        d.y_dtype = _DT[self.y_dtype or x_dtype]
        d.scale_dtype = _DT[self.w.scale.dtype]
        d.prologue = L.PROLOGUE_RMSNORM if self.gain is not None else L.PROLOGUE_NONE
        d.epilogue = (L.EPILOGUE_SILU_MUL if self.w2 is not None
                      else L.EPILOGUE_BIAS if self.bias is not None
                      else L.EPILOGUE_ADD if self.add else L.EPILOGUE_NONE)
        d.rms_eps = self.eps
        d.kernel = self.kernel
        d.split_k = self.split_k
        d.flags = self.flags
        if self.kernel_db is not None and self.kernel == L.KERNEL_AUTO and self.split_k == 0:
            from . import kernel_db as kdb
            ident = kdb.identifier(M, d.N, d.K, d.w_bits, d.group_size, d.x_dtype, d.scale_dtype, d.y_dtype,
                                   self.w2 is not None)
            hit = self.kernel_db.fetch_with_tags(ident, kdb.DEVICE_TYPE, {"fast"}, self.db_device)
            if hit is not None:
                d.kernel, d.split_k = int(hit.function["kernel"]), int(hit.function["split_k"])
        return d

    def workspace(self, d: L.LinearDesc) -> Optional[torch.Tensor]:
        key = (d.M, d.x_dtype)
        if key not in self._ws:
            n = int(self.ctx.lib.nnf_b200_linear_workspace_bytes(self.ctx.handle, ctypes.byref(d)))
            if n == 0:
                self._ws[key] = None
            else:
                ws = torch.empty(n + 256, dtype=torch.uint8, device=self.w.wq.device)
                off = (-ws.data_ptr()) % 256
                ws = ws[off:off + n]
                stream = torch.cuda.current_stream().cuda_stream
                self.ctx.check(self.ctx.lib.nnf_b200_workspace_reset(self.ctx.handle, stream, ws.data_ptr(), n))
                self._ws[key] = ws
        return self._ws[key]

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 addend: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x.dim() != 2 or x.shape[1] != self.w.K or not x.is_contiguous():
            raise ValueError(f"x must be a contiguous [M, {self.w.K}] tensor")
        M = x.shape[0]
        d = self.desc(M, x.dtype)
        if out is None:
            out = torch.empty((M, self.w.N), dtype=self.y_dtype or x.dtype, device=x.device)
        if self.add != (addend is not None):
            raise ValueError("addend must be given exactly when the node was built with add=True")
        if addend is not None and (addend.shape != out.shape or addend.dtype != out.dtype
                                   or not addend.is_contiguous()):
            raise ValueError("addend must be a contiguous [M, N] tensor of the output's dtype")
        ws = self.workspace(d)
        self.run_raw(d, x.data_ptr(), out.data_ptr(), ws, addend.data_ptr() if addend is not None else None)
        return out

    def host_entry(self, x_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
        """The call with host buffers, like the generated runtime's ``kernel_entry_host`` (``-fhost_entry``:
        ``src/nnfusion/engine/pass/codegen/cuda_codegen_pass.cpp:117-168``): copy x to the device, run the node, copy y
        back, return when y is on the host.  Both tensors must be pinned.  The three operations are captured once
        per (x, y) pair as a CUDA graph, so a call costs one graph launch and one stream synchronisation."""
        if not (x_host.is_pinned() and y_host.is_pinned()):
            raise ValueError("host_entry needs pinned host tensors")
        key = (x_host.data_ptr(), y_host.data_ptr(), tuple(x_host.shape), x_host.dtype)
        graphs = self.__dict__.setdefault("_host_graphs", {})
        if key not in graphs:
            dev = self.w.wq.device
            x_dev = torch.empty(x_host.shape, dtype=x_host.dtype, device=dev)
            y_dev = torch.empty(y_host.shape, dtype=y_host.dtype, device=dev)
            self(x_dev, out=y_dev)                  # workspace allocation and first-call set-up outside the capture
            torch.cuda.synchronize()
            stream = torch.cuda.Stream(device=dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    x_dev.copy_(x_host, non_blocking=True)
                    self(x_dev, out=y_dev)
                    y_host.copy_(y_dev, non_blocking=True)
            graphs[key] = (g, stream, x_dev, y_dev)
        g, stream, _, _ = graphs[key]
        with torch.cuda.stream(stream):
            g.replay()
        stream.synchronize()
        return y_host

    def run_raw(self, d: L.LinearDesc, x_ptr: int, y_ptr: int, ws: Optional[torch.Tensor],
                addend_ptr: Optional[int] = None) -> None:
        """The C-ABI call itself, on the current stream, with raw device addresses."""
        stream = torch.cuda.current_stream().cuda_stream
        rc = self.ctx.lib.nnf_b200_linear(
            self.ctx.handle, stream, ctypes.byref(d), x_ptr, ctypes.byref(self._abi_w),
            ctypes.byref(self._abi_w2) if self._abi_w2 is not None else None,
            self.gain.data_ptr() if self.gain is not None else None,
            self.bias.data_ptr() if self.bias is not None else addend_ptr,
            y_ptr, ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0)
        self.ctx.check(rc)
