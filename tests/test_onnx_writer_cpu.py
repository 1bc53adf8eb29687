"""The ONNX file of a dequantised linear (``nnfusion_b200/onnx_writer.py``): what is written decodes to the graph that
was meant, evaluates (by the ONNX definitions of Cast / Sub / Mul / Reshape / Gemm, in numpy) to what the oracle
computes, and folds back into the quantised weight it was written from."""
import numpy as np
import pytest

from nnfusion_b200 import onnx_writer as ow
from nnfusion_b200 import synth
from oracle import oracle as orc


def _evaluate(model, feeds):
    """A few lines of ONNX semantics: numpy broadcasting for Sub / Mul, Cast by TensorProto.DataType, Gemm with
    alpha / beta / transA / transB."""
    g = model["graph"]
    env = dict(g["initializers"])
    env.update(feeds)
    for n in g["nodes"]:
        a = [env[i] for i in n["inputs"]]
        t, at = n["op_type"], n["attrs"]
        if t == "Cast":
            out = a[0].astype({ow.FLOAT: np.float32, ow.FLOAT16: np.float16}[at["to"]])
        elif t == "Sub":
            out = a[0] - a[1]
        elif t == "Mul":
            out = a[0] * a[1]
        elif t == "Reshape":
            out = a[0].reshape(tuple(int(d) for d in a[1]))
        elif t == "Gemm":
            A = a[0].T if at.get("transA") else a[0]
            B = a[1].T if at.get("transB") else a[1]
            out = at["alpha"] * (A.astype(np.float32) @ B.astype(np.float32))
            if len(a) > 2:
                out = out + at["beta"] * a[2].astype(np.float32)
            out = out.astype(a[0].dtype)
        else:
            raise AssertionError(t)
        env[n["outputs"][0]] = out
    return env[g["outputs"][0][0]]


def test_config1_graph_per_channel_fp32(tmp_path):
    rng = np.random.Generator(np.random.PCG64(0))
    M, N, K = 16, 96, 256
    x = synth.make_x(rng, M, K, np.float32)
    w = synth.make_weights(rng, N, K, 8, K, np.float32, (0.001, 0.01), (120, 137))
    path = str(tmp_path / "config1.onnx")
    ow.write_dequant_linear(path, w, M)
    m = ow.read_model(path)
    assert m["ir_version"] == 6 and m["opset"] == 11 and m["producer"] == "nnfusion_b200"
    g = m["graph"]
    assert [n["op_type"] for n in g["nodes"]] == ["Cast", "Cast", "Sub", "Mul", "Gemm"]
    assert g["nodes"][0]["attrs"] == {"to": ow.FLOAT}
    assert g["nodes"][-1]["attrs"] == {"alpha": 1.0, "beta": 1.0, "transA": 0, "transB": 1}
    assert g["inputs"] == [("X", ow.FLOAT, (M, K))] and g["outputs"] == [("Y", ow.FLOAT, (M, N))]
    assert g["initializers"]["Wq"].dtype == np.uint8 and g["initializers"]["Wq"].shape == (N, K)
    assert g["initializers"]["scale"].shape == (N, 1) and g["initializers"]["zp"].shape == (N, 1)
    y = _evaluate(m, {"X": x})
    r = orc.linear(x, w.q, w.scale, w.zp, w.group)
    assert orc.max_rel_err(y, r) <= 1e-5
    w2, bias, M2 = ow.fold_dequant_linear(m)
    assert (M2, bias) == (M, None) and (w2.N, w2.K, w2.bits, w2.group) == (N, K, 8, K)
    np.testing.assert_array_equal(w2.q, w.q)
    np.testing.assert_array_equal(w2.zp, w.zp)
    np.testing.assert_array_equal(w2.scale, w.scale)


def test_grouped_uint4_fp16_with_bias(tmp_path):
    rng = np.random.Generator(np.random.PCG64(1))
    M, N, K = 3, 48, 512
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    bias = rng.standard_normal(N).astype(np.float16)
    data = ow.model(ow.dequant_linear_graph(w, M, np.float16, bias))
    m = ow.read_model(data)
    ops = [n["op_type"] for n in m["graph"]["nodes"]]
    assert ops == ["Reshape", "Cast", "Cast", "Sub", "Mul", "Reshape", "Gemm"]
    assert m["graph"]["initializers"]["zp"].shape == (N, K // 128, 1)
    y = _evaluate(m, {"X": x})
    r = orc.linear(x, w.q, w.scale, w.zp, w.group, bias=bias.astype(np.float32))
    assert orc.max_rel_err(y, r) <= 5e-3
    w2, b2, _ = ow.fold_dequant_linear(m, bits=4)
    assert (w2.bits, w2.group) == (4, 128)
    np.testing.assert_array_equal(w2.wq, w.wq)            # packs to the same bytes the kernels read
    np.testing.assert_array_equal(w2.zpq, w.zpq)
    np.testing.assert_array_equal(b2, bias)


def test_other_graphs_are_not_folded():
    rng = np.random.Generator(np.random.PCG64(2))
    w = synth.make_weights(rng, 16, 128, 8, 128, np.float32, (0.001, 0.01), (120, 137))
    g = ow.dequant_linear_graph(w, 2)
    m = ow.read_model(ow.model(g))
    m["graph"]["nodes"][-1]["attrs"]["transB"] = 0
    with pytest.raises(ValueError):
        ow.fold_dequant_linear(m)
    m = ow.read_model(ow.model(g))
    with pytest.raises(ValueError):
        ow.fold_dequant_linear(m, bits=4)                 # values above 15 cannot be packed


def test_varints_round_trip():
    for v in (0, 1, 127, 128, 300, 2**31, 2**40 + 5):
        (f, wire, got), = list(ow._fields(ow._int(3, v)))
        assert (f, wire, got) == (3, 0, v)
