"""On-disk container of the quantised weights, in the reference's own conventions, and its loader.

The reference dumps every ``Constant`` node's bytes to ``./Constant/<tensor name>.bin`` at compile time and reads
the files back in ``cuda_init`` through a heap buffer and ``cudaMemcpyAsync``
(``src/nnfusion/core/kernels/cuda_gpu/kernels/constant.cpp:36-59``); ``para_info.json`` lists the graph's tensors as
``{"weight": {<frontend name>: {"name", "id": "((<dtype>*)(...))", "shape"}}}``
(``src/nnfusion/engine/pass/extract_graph_signature.cpp:150-236``) with the dtype names of
``src/python/nnfusion/dtypes.py:12-46``.  That table has no 4-bit entry, so packed uint4 tensors travel as ``uint8``
of shape ``[N, K/2]`` (zero-points ``[N, ceil(K/g/2)]``); the logical format is recorded next to them under a
``"quant"`` key that the reference's parser ignores.

Layout written here, for a linear called ``name``::

    <dir>/Constant/<name>.wq.bin      uint8  [N, K/2] (uint4, low nibble = even k) or [N, K]
    <dir>/Constant/<name>.scale.bin   half / float [N, K/g]
    <dir>/Constant/<name>.zp.bin      uint8, packed like the weights along the group axis
    <dir>/para_info.json

Files are raw row-major bytes exactly as the kernels read them: loading is ``numpy.memmap`` -> pinned staging ->
one asynchronous copy per tensor, no re-layout.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import numpy as np

from .synth import QuantLinear

_DTYPE_NAME = {np.dtype(np.uint8): "uint8", np.dtype(np.float16): "half", np.dtype(np.float32): "float"}
_NAME_DTYPE = {"uint8": np.uint8, "half": np.float16, "float16": np.float16, "float": np.float32,
               "float32": np.float32}


def _entry(tensor_name: str, arr: np.ndarray, index: int) -> dict:
    return {"name": tensor_name, "id": f"(({_DTYPE_NAME[arr.dtype]}*)(inputs[{index}]))", "shape": list(arr.shape)}


def _load_info(directory: str) -> dict:
    path = os.path.join(directory, "para_info.json")
    if not os.path.exists(path):
        return {"input": {}, "weight": {}, "output": {}}
    with open(path) as f:
        return json.load(f)


def save_linear(directory: str, name: str, w: QuantLinear) -> Dict[str, str]:
    """Write one quantised linear and register its three tensors in ``para_info.json``; returns the file paths."""
    const_dir = os.path.join(directory, "Constant")
    os.makedirs(const_dir, exist_ok=True)
    info = _load_info(directory)
    weights = info.setdefault("weight", {})
    paths = {}
    base = len(weights)
    for k, (suffix, arr) in enumerate((("wq", w.wq), ("scale", w.scale), ("zp", w.zpq))):
        arr = np.ascontiguousarray(arr)
        tensor = f"{name}.{suffix}"
        path = os.path.join(const_dir, tensor + ".bin")
        with open(path, "wb") as f:          # the same raw dump Constant::emit_function_body writes
            f.write(arr.tobytes())
        weights[tensor] = _entry(tensor, arr, base + k)
        paths[suffix] = path
    info.setdefault("quant", {})[name] = {"N": w.N, "K": w.K, "w_bits": w.bits, "group_size": w.group}
    with open(os.path.join(directory, "para_info.json"), "w") as f:
        json.dump(info, f, indent=4)
    return paths


def _dtype_of(entry: dict):
    # the reference's executor strips the dtype out of "id" the same way (src/python/nnfusion/executor.py:30-67)
    ident = entry["id"]
    name = ident[ident.index("((") + 2: ident.index("*")]
    if name not in _NAME_DTYPE:
        raise ValueError(f"dtype {name!r} of tensor {entry['name']!r} is not one this library reads")
    return np.dtype(_NAME_DTYPE[name])


def open_tensor(directory: str, tensor: str) -> np.ndarray:
    """Memory-map one constant; checks the file size against the recorded shape."""
    info = _load_info(directory)
    if tensor not in info.get("weight", {}):
        raise KeyError(f"{tensor!r} is not listed in para_info.json")
    entry = info["weight"][tensor]
    dtype, shape = _dtype_of(entry), tuple(entry["shape"])
    path = os.path.join(directory, "Constant", entry["name"] + ".bin")
    want = int(np.prod(shape)) * dtype.itemsize
    have = os.path.getsize(path)
    if have != want:
        raise ValueError(f"{path}: {have} bytes on disk, {want} expected for {dtype.name}{list(shape)}")
    if want == 0:
        return np.zeros(shape, dtype)
    return np.memmap(path, dtype=dtype, mode="r", shape=shape)


def load_linear_host(directory: str, name: str) -> QuantLinear:
    """The host-side view (memory-mapped, nothing copied until it is read)."""
    info = _load_info(directory)
    if name not in info.get("quant", {}):
        raise KeyError(f"no quantised linear called {name!r}")
    q = info["quant"][name]
    wq, scale, zpq = (open_tensor(directory, f"{name}.{s}") for s in ("wq", "scale", "zp"))
    N, K, bits, group = q["N"], q["K"], q["w_bits"], q["group_size"]
    G = K // group
    if wq.shape != (N, K // 2 if bits == 4 else K) or scale.shape != (N, G) or \
            zpq.shape != (N, (G + 1) // 2 if bits == 4 else G):
        raise ValueError(f"{name}: tensor shapes do not match N={N}, K={K}, {bits} bits, groups of {group}")
    return QuantLinear.from_packed(N, K, bits, group, wq, scale, zpq)


def load_linear(directory: str, name: str, device: str = "cuda:0", stream=None):
    """Upload one linear: memory-map -> pinned staging -> asynchronous copy, tensor by tensor; returns a
    ``DeviceWeight``.  The bytes on disk are the bytes the kernels read: there is no re-layout step."""
    import torch

    from .linear import DeviceWeight

    w = load_linear_host(directory, name)
    out = []
    with torch.cuda.stream(stream) if stream is not None else _null():
        for arr in (w.wq, w.scale, w.zpq):
            staged = torch.from_numpy(np.array(arr)).pin_memory()   # (a writable copy of the read-only mapping)
            out.append(staged.to(device, non_blocking=True))
    torch.cuda.current_stream().synchronize() if stream is None else stream.synchronize()
    return DeviceWeight(w.N, w.K, w.bits, w.group, *out)


class _null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False
