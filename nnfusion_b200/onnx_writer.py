"""Writes the ONNX file of a dequantised linear the way an exporter spells it,

    Y = X . ((Cast(Wq) - Cast(zp)) * scale)^T   ==   Cast -> Sub -> Mul -> Gemm(transB = 1)

without the ``onnx`` package (not installed here): a small protocol-buffer encoder for the handful of messages
involved, following the schema the reference vendors (``thirdparty/onnx/proto/onnx/onnx-ml.proto``: ``ModelProto``,
``GraphProto``, ``NodeProto``, ``AttributeProto``, ``TensorProto``, ``ValueInfoProto``, ``TypeProto``).  This is the
graph of the first benchmark configuration -- what ``nnfusion model.onnx -f onnx`` imports (``Cast``:
``src/nnfusion/frontend/onnx_import/op/cast.hpp:35-51``; ``Sub`` / ``Mul`` with numpy broadcasting:
``op/binaryop.hpp:89-107``; ``Gemm``: ``op/gemm.cpp``) and what the plugin's fold pass turns into one ``DequantDot``.

For weights in groups along K (not expressible by a [N,1] broadcast) the file carries the rank-3 form
``Reshape([N,G,g]) -> Cast -> Sub([N,G,1]) -> Mul([N,G,1]) -> Reshape([N,K])`` in front of the Gemm.  Packed uint4
weights are written unpacked, one uint8 per element: ONNX at this schema version has no 4-bit element type.

:func:`read_model` decodes such a file again (for tests and for :mod:`nnfusion_b200.jit`).
"""
from __future__ import annotations

import struct
from typing import Dict, List, Optional, Tuple

import numpy as np

from .synth import QuantLinear

# TensorProto.DataType
FLOAT, UINT8, INT64, FLOAT16 = 1, 2, 7, 10
_NP_OF = {FLOAT: np.float32, UINT8: np.uint8, INT64: np.int64, FLOAT16: np.float16}
_DT_OF = {np.dtype(np.float32): FLOAT, np.dtype(np.uint8): UINT8, np.dtype(np.int64): INT64,
          np.dtype(np.float16): FLOAT16}
# AttributeProto.AttributeType
ATTR_FLOAT, ATTR_INT, ATTR_INTS = 1, 2, 7


# ------------------------------------------------------------------------------------------------ wire format
def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _int(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(v)


def _bytes(field: int, payload: bytes) -> bytes:
    return _key(field, 2) + _varint(len(payload)) + payload


def _str(field: int, s: str) -> bytes:
    return _bytes(field, s.encode("utf-8"))


def _f32(field: int, v: float) -> bytes:
    return _key(field, 5) + struct.pack("<f", v)


# ------------------------------------------------------------------------------------------------ messages
def tensor(name: str, arr: np.ndarray) -> bytes:
    arr = np.ascontiguousarray(arr)
    out = b"".join(_int(1, d) for d in arr.shape) + _int(2, _DT_OF[arr.dtype]) + _str(8, name)
    return out + _bytes(9, arr.tobytes())                       # raw_data, little endian


def value_info(name: str, elem_type: int, shape) -> bytes:
    dims = b"".join(_bytes(1, _int(1, int(d))) for d in shape)  # TensorShapeProto.dim { dim_value }
    ttype = _int(1, elem_type) + _bytes(2, dims)                # TypeProto.Tensor { elem_type, shape }
    return _str(1, name) + _bytes(2, _bytes(1, ttype))          # ValueInfoProto { name, type { tensor_type } }


def attribute(name: str, value) -> bytes:
    if isinstance(value, float):
        return _str(1, name) + _f32(2, value) + _int(20, ATTR_FLOAT)
    if isinstance(value, int):
        return _str(1, name) + _int(3, value) + _int(20, ATTR_INT)
    return _str(1, name) + b"".join(_int(8, int(v)) for v in value) + _int(20, ATTR_INTS)


def node(op_type: str, inputs: List[str], outputs: List[str], name: str = "", **attrs) -> bytes:
    out = b"".join(_str(1, i) for i in inputs) + b"".join(_str(2, o) for o in outputs)
    out += _str(3, name or outputs[0]) + _str(4, op_type)
    return out + b"".join(_bytes(5, attribute(k, v)) for k, v in attrs.items())


def model(graph: bytes, opset: int = 11, producer: str = "nnfusion_b200") -> bytes:
    return _int(1, 6) + _str(2, producer) + _bytes(7, graph) + _bytes(8, _str(1, "") + _int(2, opset))


# ------------------------------------------------------------------------------------------------ the graph
def dequant_linear_graph(w: QuantLinear, M: int, x_dtype=np.float32, bias: Optional[np.ndarray] = None,
                         name: str = "dequant_linear") -> bytes:
    """GraphProto bytes of Y[M,N] = X[M,K] . dequant(W)^T (+ bias); X is the only graph input, everything else an
    initializer.  Scales are written in X's element type (every operand of an element-wise ONNX node has one type)."""
    xt = np.dtype(x_dtype)
    et = _DT_OF[xt]
    G = w.K // w.group
    nodes, inits = [], []
    inits.append(tensor("Wq", w.q.astype(np.uint8)))
    if G == 1:
        inits.append(tensor("zp", w.zp.reshape(w.N, 1).astype(np.uint8)))
        inits.append(tensor("scale", w.scale.reshape(w.N, 1).astype(xt)))
        nodes.append(node("Cast", ["Wq"], ["Wq_f"], to=et))
        nodes.append(node("Cast", ["zp"], ["zp_f"], to=et))
        nodes.append(node("Sub", ["Wq_f", "zp_f"], ["W_centered"]))
        nodes.append(node("Mul", ["W_centered", "scale"], ["W_dq"]))
    else:
        inits.append(tensor("zp", w.zp.reshape(w.N, G, 1).astype(np.uint8)))
        inits.append(tensor("scale", w.scale.reshape(w.N, G, 1).astype(xt)))
        inits.append(tensor("shape_grouped", np.array([w.N, G, w.group], np.int64)))
        inits.append(tensor("shape_flat", np.array([w.N, w.K], np.int64)))
        nodes.append(node("Reshape", ["Wq", "shape_grouped"], ["Wq_g"]))
        nodes.append(node("Cast", ["Wq_g"], ["Wq_f"], to=et))
        nodes.append(node("Cast", ["zp"], ["zp_f"], to=et))
        nodes.append(node("Sub", ["Wq_f", "zp_f"], ["W_centered"]))
        nodes.append(node("Mul", ["W_centered", "scale"], ["W_dq_g"]))
        nodes.append(node("Reshape", ["W_dq_g", "shape_flat"], ["W_dq"]))
    gemm_in = ["X", "W_dq"]
    if bias is not None:
        inits.append(tensor("bias", np.asarray(bias).astype(xt)))
        gemm_in.append("bias")
    nodes.append(node("Gemm", gemm_in, ["Y"], alpha=1.0, beta=1.0, transA=0, transB=1))
    g = b"".join(_bytes(1, n) for n in nodes) + _str(2, name) + b"".join(_bytes(5, t) for t in inits)
    g += _bytes(11, value_info("X", et, (M, w.K))) + _bytes(12, value_info("Y", et, (M, w.N)))
    return g


def write_dequant_linear(path: str, w: QuantLinear, M: int, x_dtype=np.float32, bias=None) -> None:
    with open(path, "wb") as f:
        f.write(model(dequant_linear_graph(w, M, x_dtype, bias)))


# ------------------------------------------------------------------------------------------------ reading back
def _fields(buf: bytes):
    """Yields (field number, wire type, value) of one message; length-delimited values as bytes."""
    i, n = 0, len(buf)
    while i < n:
        key, shift = 0, 0
        while True:
            b = buf[i]
            i += 1
            key |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                break
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, shift = 0, 0
            while True:
                b = buf[i]
                i += 1
                v |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            yield field, wire, v
        elif wire == 2:
            ln, shift = 0, 0
            while True:
                b = buf[i]
                i += 1
                ln |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            yield field, wire, bytes(buf[i:i + ln])
            i += ln
        elif wire == 5:
            yield field, wire, struct.unpack("<f", buf[i:i + 4])[0]
            i += 4
        elif wire == 1:
            yield field, wire, struct.unpack("<d", buf[i:i + 8])[0]
            i += 8
        else:
            raise ValueError(f"wire type {wire} is not used by the messages this module reads")


def _read_tensor(buf: bytes) -> Tuple[str, np.ndarray]:
    dims, dt, name, raw = [], None, "", b""
    for f, _, v in _fields(buf):
        if f == 1:
            dims.append(v)
        elif f == 2:
            dt = v
        elif f == 8:
            name = v.decode()
        elif f == 9:
            raw = v
    return name, np.frombuffer(raw, dtype=_NP_OF[dt]).reshape(dims).copy()


def _read_node(buf: bytes) -> dict:
    n = {"inputs": [], "outputs": [], "name": "", "op_type": "", "attrs": {}}
    for f, _, v in _fields(buf):
        if f == 1:
            n["inputs"].append(v.decode())
        elif f == 2:
            n["outputs"].append(v.decode())
        elif f == 3:
            n["name"] = v.decode()
        elif f == 4:
            n["op_type"] = v.decode()
        elif f == 5:
            name, val, ints = "", None, []
            for af, _, av in _fields(v):
                if af == 1:
                    name = av.decode()
                elif af in (2, 3):
                    val = av
                elif af == 8:
                    ints.append(av)
            n["attrs"][name] = ints if ints else val
    return n


def _read_value_info(buf: bytes) -> Tuple[str, int, Tuple[int, ...]]:
    name, elem, shape = "", 0, []
    for f, _, v in _fields(buf):
        if f == 1:
            name = v.decode()
        elif f == 2:
            for tf, _, tv in _fields(v):
                if tf == 1:                     # tensor_type
                    for ef, _, ev in _fields(tv):
                        if ef == 1:
                            elem = ev
                        elif ef == 2:
                            for df, _, dv in _fields(ev):
                                if df == 1:
                                    shape.extend(val for f2, _, val in _fields(dv) if f2 == 1)
    return name, elem, tuple(shape)


def read_model(path_or_bytes) -> dict:
    """``{"ir_version", "opset", "producer", "graph": {"name", "nodes", "initializers", "inputs", "outputs"}}``."""
    data = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    out = {"ir_version": None, "opset": None, "producer": "", "graph": None}
    for f, _, v in _fields(data):
        if f == 1:
            out["ir_version"] = v
        elif f == 2:
            out["producer"] = v.decode()
        elif f == 8:
            out["opset"] = dict((ff, vv) for ff, _, vv in _fields(v)).get(2)
        elif f == 7:
            g = {"name": "", "nodes": [], "initializers": {}, "inputs": [], "outputs": []}
            for gf, _, gv in _fields(v):
                if gf == 1:
                    g["nodes"].append(_read_node(gv))
                elif gf == 2:
                    g["name"] = gv.decode()
                elif gf == 5:
                    name, arr = _read_tensor(gv)
                    g["initializers"][name] = arr
                elif gf == 11:
                    g["inputs"].append(_read_value_info(gv))
                elif gf == 12:
                    g["outputs"].append(_read_value_info(gv))
            out["graph"] = g
    return out


def fold_dequant_linear(m: dict, bits: int = 8) -> Tuple[QuantLinear, Optional[np.ndarray], int]:
    """What the plugin's fold pass does to the imported graph, on the decoded file: matches
    Gemm(transB) <- Mul <- Sub <- Cast (with the optional Reshapes of the grouped form), checks the broadcast shapes
    and returns the quantised weight, the bias (or None) and M.  Raises ValueError on any other graph.  ``bits`` = 4
    packs the weights again (the caller knows they were uint4: the file cannot say so); values are checked."""
    g = m["graph"]
    by_out: Dict[str, dict] = {o: n for n in g["nodes"] for o in n["outputs"]}
    init = g["initializers"]

    def producer(name, op):
        n = by_out.get(name)
        if n is None or n["op_type"] != op:
            raise ValueError(f"expected {op} producing {name}")
        return n

    def skip_reshape(name):
        n = by_out.get(name)
        return skip_reshape(n["inputs"][0]) if n is not None and n["op_type"] == "Reshape" else name

    gemm = next((n for n in g["nodes"] if n["op_type"] == "Gemm"), None)
    if gemm is None or gemm["attrs"].get("transB") != 1 or gemm["attrs"].get("transA", 0) != 0:
        raise ValueError("no Gemm with transB = 1")
    mul = producer(skip_reshape(gemm["inputs"][1]), "Mul")
    scale_name = next(i for i in mul["inputs"] if i in init)
    sub = producer(next(i for i in mul["inputs"] if i not in init), "Sub")
    wq_name = skip_reshape(producer(sub["inputs"][0], "Cast")["inputs"][0])
    zp_name = skip_reshape(producer(sub["inputs"][1], "Cast")["inputs"][0])
    wq, zp, scale = init[wq_name], init[zp_name], init[scale_name]
    if wq.dtype != np.uint8 or zp.dtype != np.uint8 or wq.ndim != 2:
        raise ValueError("weights and zero-points must be uint8 initializers")
    N, K = wq.shape
    if zp.shape != scale.shape or zp.shape[0] != N or zp.shape[-1] != 1:
        raise ValueError("scale and zero-point must broadcast along the innermost axis")
    G = 1 if zp.ndim == 2 else zp.shape[1]
    if bits not in (4, 8) or (bits == 4 and (int(wq.max(initial=0)) > 15 or int(zp.max(initial=0)) > 15)):
        raise ValueError("bits must be 8, or 4 with every weight and zero-point below 16")
    w = QuantLinear(N, K, bits, K // G, wq, scale.reshape(N, G), zp.reshape(N, G))
    bias = init[gemm["inputs"][2]] if len(gemm["inputs"]) > 2 else None
    (_, _, xshape), = g["inputs"]
    return w, bias, int(xshape[0])
