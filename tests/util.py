"""Shared helpers of the GPU parity tests: run one linear through the C-ABI, and through the oracle."""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc

TOL_F32 = 1e-3   # max|y - r| / max|r| for fp32 paths
TOL_F16 = 5e-3   # for fp16 paths


def oracle_linear(x, w, w2=None, gain=None, bias=None, eps=1e-6, out_dtype=None):
    return orc.linear(x, w.q, w.scale, w.zp, w.group,
                      q2=None if w2 is None else w2.q, scale2=None if w2 is None else w2.scale,
                      zp2=None if w2 is None else w2.zp, gain=gain, eps=eps, bias=bias,
                      out_dtype=out_dtype)


def gpu_linear(x, w, w2=None, gain=None, bias=None, eps=1e-6, out_dtype=None, kernel=0, split_k=0,
               repeat=1, return_op=False, flags=0):
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    dev = "cuda:0"
    dw = DeviceWeight.from_host(w, dev)
    dw2 = DeviceWeight.from_host(w2, dev) if w2 is not None else None
    tg = torch.from_numpy(np.ascontiguousarray(gain, np.float32)).to(dev) if gain is not None else None
    tb = torch.from_numpy(np.ascontiguousarray(bias, np.float32)).to(dev) if bias is not None else None
    ydt = None
    if out_dtype is not None:
        ydt = torch.float16 if np.dtype(out_dtype) == np.float16 else torch.float32
    op = DequantDot(dw, dw2, gain=tg, bias=tb, eps=eps, y_dtype=ydt, kernel=kernel, split_k=split_k, flags=flags)
    tx = torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    outs = []
    for _ in range(repeat):
        y = op(tx)
        torch.cuda.synchronize()
        outs.append(y.cpu().numpy())
    op.ctx.device_status()   # no bounded wait inside the kernels may have given up
    if return_op:
        return outs, op
    return outs[0] if repeat == 1 else outs


def tol_for(x, w):
    return TOL_F32 if (x.dtype == np.float32 and w.scale.dtype == np.float32) else TOL_F16
