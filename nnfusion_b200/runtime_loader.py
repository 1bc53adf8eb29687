"""Loads a generated ``nnfusion_rt`` directory the way NNFusion's Python ``Executor`` does and runs its
``kernel_entry``.

The behaviour follows ``src/python/nnfusion/executor.py`` of the reference step by step (cited per function), written
afresh because the reference package is not importable where this library runs:

* the shared object is the file in the directory whose name starts with ``libnnf`` and ends with ``rt.so`` (``:14-27``);
* ``kernel_entry_host`` is preferred over ``kernel_entry`` when the runtime exports it (``:106-111``);
* ``get_device_type()`` picks the init / free pair, ``cuda_init`` / ``cuda_free`` for 0 (``:77-84,112-118``), and the
  init function runs with the runtime directory as working directory, because ``cuda_init`` opens ``Constant/*.bin``
  by relative path (``:120-127``); a non-zero ``get_workspace_size()`` makes the caller reserve that many bytes and
  pass the pointer to init (``:230-243``);
* ``para_info.json`` gives, per frontend name, the tensor's name, its position and C type inside the text
  ``"((<type>*)(inputs[<i>]))"`` and its shape (``:30-67``); weights and inputs share the ``inputs[...]`` numbering;
* a call checks every fed tensor's shape and element type against that description and passes raw pointers,
  inputs first, then outputs (``:171-228``).

One deviation, marked below: the reference leaves the C type ``half`` as the string ``"half"``, which never equals the
``"float16"`` its tensor wrappers report; here it is normalised to ``"float16"`` so that fp16 graphs can be fed.
"""
from __future__ import annotations

import contextlib
import ctypes
import json
import os
from dataclasses import dataclass
from typing import Dict, Sequence, Tuple

# dtype string -> ctypes element type (src/python/nnfusion/dtypes.py:12-46; fp16 travels as 16-bit words there too)
_CTYPE = {"float16": ctypes.c_uint16, "float32": ctypes.c_float, "float64": ctypes.c_double, "int8": ctypes.c_int8,
          "int16": ctypes.c_int16, "int32": ctypes.c_int32, "int64": ctypes.c_int64, "uint8": ctypes.c_uint8}

_INIT_FREE = {0: ("cuda_init", "cuda_free"), 1: ("rocm_init", "rocm_free"), 2: ("cpu_init", "cpu_free"),
              3: ("hlsl_init", "hlsl_free"), 4: ("graphcore_init", "graphcore_free")}


@dataclass(frozen=True)
class TensorInfo:
    """What ``para_info.json`` says about one input or output (the reference's ``IODescription``)."""
    name: str
    index: int
    dtype: str
    shape: Tuple[int, ...]
    tensor_name: str


@dataclass
class Fed:
    """A tensor as the executor is fed with it: address, element pointer type, shape, dtype string, and the object
    that owns the memory (the reference's ``DataFormat``, ``data_format.py:9-49``)."""
    pointer: object
    pointer_type: object
    shape: Tuple[int, ...]
    dtype: str
    owner: object = None


def feed_torch(t) -> Fed:
    """``cast_pytorch_tensor`` (``data_format.py:52-64``): contiguous tensors only; device or (pinned) host memory."""
    if not t.is_contiguous():
        raise ValueError("only contiguous tensors can be fed")
    dtype = str(t.dtype).split(".")[-1]
    ptype = ctypes.POINTER(_CTYPE[dtype])
    return Fed(ctypes.cast(t.data_ptr(), ptype), ptype, tuple(t.shape) or (1,), dtype, t)


def feed_numpy(a) -> Fed:
    """``cast_numpy_array`` (``data_format.py:67-74``)."""
    ptype = ctypes.POINTER(_CTYPE[a.dtype.name])
    return Fed(a.ctypes.data_as(ptype), ptype, tuple(a.shape) or (1,), a.dtype.name, a)


def find_runtime_library(rt_dir: str) -> str:
    for entry in sorted(os.listdir(rt_dir)):
        if entry.startswith("libnnf") and entry.endswith("rt.so"):
            return os.path.join(rt_dir, entry)
    raise FileNotFoundError(f"no libnnf*rt.so in {rt_dir}")


def _dtype_of(c_type: str) -> str:
    if c_type.endswith("_t"):
        return c_type[:-2]
    if c_type == "half":          # deviation from the reference, see the module's docstring
        return "float16"
    return {"float": "float32", "double": "float64"}.get(c_type, c_type)


def read_para_info(path: str):
    """Returns (weights, inputs, outputs): dictionaries frontend name -> :class:`TensorInfo`."""
    with open(path) as f:
        doc = json.load(f)

    def section(key: str, marker: str) -> Dict[str, TensorInfo]:
        out = {}
        for name, entry in doc.get(key, {}).items():
            ident = entry["id"]                       # e.g. "((float*)(inputs[0]))"
            index = int(ident.split(marker)[1].split("]")[0])
            c_type = ident[2:].split("*")[0]
            shape = tuple(entry["shape"]) or (1,)
            out[name] = TensorInfo(name, index, _dtype_of(c_type), shape, entry["name"])
        return out

    return section("weight", "inputs["), section("input", "inputs["), section("output", "outputs[")


@contextlib.contextmanager
def _working_directory(path: str):
    before = os.getcwd()
    os.chdir(path)
    try:
        yield
    finally:
        os.chdir(before)


class RuntimeExecutor:
    """``Executor(nnf_rt_dir)``: load, initialise, describe, call, free."""

    def __init__(self, rt_dir: str, reserve=None):
        """``reserve(n_bytes) -> (pointer, owner)`` is asked for device memory when the runtime wants a workspace
        from its caller (``get_workspace_size() > 0``); runtimes generated by this package never do."""
        rt_dir = os.path.abspath(rt_dir)
        self.library_path = find_runtime_library(rt_dir)
        self.lib = ctypes.cdll.LoadLibrary(self.library_path)
        self.host_entry = hasattr(self.lib, "kernel_entry_host")
        if self.host_entry:
            self.entry = self.lib.kernel_entry_host
        elif hasattr(self.lib, "kernel_entry"):
            self.entry = self.lib.kernel_entry
        else:
            raise RuntimeError("the runtime exports neither kernel_entry_host nor kernel_entry")
        if not hasattr(self.lib, "get_device_type"):
            raise RuntimeError("the runtime exports no get_device_type")
        self.lib.get_device_type.restype = ctypes.c_int
        self.device_type = self.lib.get_device_type()
        if self.device_type not in _INIT_FREE:
            raise RuntimeError(f"unknown device type {self.device_type}")
        init_name, free_name = _INIT_FREE[self.device_type]
        self._free = getattr(self.lib, free_name, None)
        self._initialised = False
        init = getattr(self.lib, init_name, None)
        if init is not None:
            with _working_directory(rt_dir):
                size_fn = getattr(self.lib, "get_workspace_size", None)
                n_bytes = 0
                if size_fn is not None:
                    size_fn.restype = ctypes.c_int64
                    n_bytes = int(size_fn())
                if n_bytes:
                    if reserve is None:
                        raise RuntimeError(f"the runtime asks its caller for {n_bytes} bytes of workspace")
                    pointer, self._workspace_owner = reserve(n_bytes)
                    init(pointer)
                else:
                    init()
            self._initialised = True
        weights, inputs, outputs = read_para_info(os.path.join(rt_dir, "para_info.json"))
        fed_side = [None] * (len(weights) + len(inputs))
        for info in list(weights.values()) + list(inputs.values()):
            fed_side[info.index] = info
        out_side = [None] * len(outputs)
        for info in outputs.values():
            out_side[info.index] = info
        if None in fed_side or None in out_side:
            raise RuntimeError("para_info.json leaves an input or output position undescribed")
        self.inputs: Sequence[TensorInfo] = tuple(fed_side)
        self.outputs: Sequence[TensorInfo] = tuple(out_side)
        self._in_pos = {i.name: i.index for i in fed_side}
        self._out_pos = {o.name: o.index for o in out_side}

    def close(self):
        if self._initialised and self._free is not None:
            self._free()
        self._initialised = False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __call__(self, inputs: Dict[str, Fed], outputs: Dict[str, Fed], strict: bool = True):
        """Runs the entry point on the named tensors; raises on unknown names (``strict``), on shape or type
        mismatches and on positions left unfed."""
        n_in = len(self.inputs)
        types = [None] * (n_in + len(self.outputs))
        values = [None] * (n_in + len(self.outputs))
        for side, table, described, base in ((inputs, self._in_pos, self.inputs, 0),
                                             (outputs, self._out_pos, self.outputs, n_in)):
            for name, fed in side.items():
                if name not in table:
                    if strict:
                        raise KeyError(f"the runtime has no tensor named {name}")
                    continue
                want = described[table[name]]
                if tuple(fed.shape) != want.shape or fed.dtype != want.dtype:
                    raise TypeError(f"{name}: expected {want.shape} {want.dtype}, fed {tuple(fed.shape)} {fed.dtype}")
                types[base + table[name]] = fed.pointer_type
                values[base + table[name]] = fed.pointer
        if None in values:
            raise ValueError("an input or output of the runtime was not fed")
        self.entry.argtypes = types
        return self.entry(*values)
