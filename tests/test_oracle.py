"""Pins the CPU oracle: against the reference's own known-answer vectors, against the
reference's MLAS compiled in place (when built), and its three restatements against
one another."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.golden import reference_vectors as gv
from nnfusion_b200 import synth

needs_ref = pytest.mark.skipif(not orc.have_ref(), reason="oracle/_ref not built")


def _dot_as_2d(a_shape, b_shape, axes, a, b):
    a = np.asarray(a, np.float32).reshape(a_shape)
    b = np.asarray(b, np.float32).reshape(b_shape)
    if axes == 0:
        return a.reshape(-1, 1), b.reshape(1, -1)
    K = b_shape[0]
    return a.reshape(-1, K), b.reshape(K, -1)


@pytest.mark.parametrize("case", gv.DOT_INVENTORY, ids=lambda c: f"dot{c[0]}")
def test_dot_inventory(case):
    _, a_shape, b_shape, axes, a, b, want = case
    a2, b2 = _dot_as_2d(a_shape, b_shape, axes, a, b)
    want = np.asarray(want, np.float32)
    got = orc.c_dot(a2, b2, trans_b=False)
    np.testing.assert_array_equal(got.ravel(), want)          # small integers: exact
    got_t = orc.c_dot(a2, np.ascontiguousarray(b2.T), trans_b=True, naive=False)
    np.testing.assert_array_equal(got_t.ravel(), want)
    if orc.have_ref():
        np.testing.assert_array_equal(orc.ref_sgemm(a2, b2).ravel(), want)


def test_gemm_op():
    g = gv.GEMM_OP
    a = np.asarray(g["a"], np.float32).reshape(g["a_shape"])
    b = np.asarray(g["b"], np.float32).reshape(g["b_shape"])
    c = np.asarray(g["c"], np.float32)
    want = np.asarray(g["y"], np.float32).reshape(g["y_shape"])
    # importer: Dot(transA, transB) -> Multiply(alpha) -> Add(beta * C)
    d = orc.c_dot(np.ascontiguousarray(a.T), b, trans_b=True)
    got = d * np.float32(g["alpha"]) + np.float32(g["beta"]) * c[None, :]
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-6)   # vectors are printed to 6 digits
    if orc.have_ref():
        r = orc.ref_sgemm(a, b, trans_a=True, trans_b=True)
        np.testing.assert_allclose(r * np.float32(g["alpha"]) + np.float32(g["beta"]) * c[None, :],
                                   want, rtol=0, atol=2e-6)


@pytest.mark.parametrize("case", gv.MATMUL_OPS, ids=lambda c: c[0])
def test_matmul_ops(case):
    _, a_shape, b_shape, want = case
    a = np.arange(int(np.prod(a_shape)), dtype=np.float32).reshape(a_shape)
    b = np.arange(int(np.prod(b_shape)), dtype=np.float32).reshape(b_shape)
    want = np.asarray(want, np.float32)
    # numpy broadcasting of the batch dims, each 2-D product through the oracle Dot
    a_ = a if a.ndim > 1 else a[None, :]
    b_ = b if b.ndim > 1 else b[:, None]
    batch = np.broadcast_shapes(a_.shape[:-2], b_.shape[:-2])
    ab = np.broadcast_to(a_, batch + a_.shape[-2:]).reshape((-1,) + a_.shape[-2:])
    bb = np.broadcast_to(b_, batch + b_.shape[-2:]).reshape((-1,) + b_.shape[-2:])
    outs = [orc.c_dot(np.ascontiguousarray(x), np.ascontiguousarray(y), trans_b=False)
            for x, y in zip(ab, bb)]
    np.testing.assert_array_equal(np.concatenate([o.ravel() for o in outs]), want)


def test_elementwise_inventory():
    L = orc.lib()
    for fn, (a, b, want) in (("orc_subtract_f32", gv.SUBTRACT), ("orc_multiply_f32", gv.MULTIPLY)):
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        out = np.empty_like(a)
        getattr(L, fn)(orc._ptr(a, orc._F), orc._ptr(b, orc._F), orc._ptr(out, orc._F), a.size)
        np.testing.assert_array_equal(out, np.asarray(want, np.float32))


def test_u4_pack_roundtrip():
    rng = np.random.default_rng(1)
    v = rng.integers(0, 16, size=(5, 14), dtype=np.uint8)
    p = orc.np_pack_u4(v)
    assert p.shape == (5, 7)
    np.testing.assert_array_equal(orc.np_unpack_u4(p), v)
    out = np.empty(v.size, np.uint8)
    orc.lib().orc_unpack_u4(orc._ptr(p, orc._U8), orc._ptr(out, orc._U8), v.size)
    np.testing.assert_array_equal(out.reshape(v.shape), v)
    assert p[0, 0] == (v[0, 0] | (v[0, 1] << 4))


def test_f16_conversions_match_numpy():
    rng = np.random.default_rng(2)
    f = (rng.standard_normal(4096) * 10 ** rng.uniform(-6, 4, 4096)).astype(np.float32)
    np.testing.assert_array_equal(orc.c_f32_to_f16(f).view(np.uint16), f.astype(np.float16).view(np.uint16))
    h = f.astype(np.float16)
    np.testing.assert_array_equal(orc.c_f16_to_f32(h), h.astype(np.float32))


@pytest.mark.parametrize("bits,group", [(8, 256), (8, 64), (4, 128)])
def test_dequant_c_equals_numpy(bits, group):
    rng = np.random.Generator(np.random.PCG64(3))
    w = synth.make_weights(rng, 24, 256, bits, group, np.float32 if bits == 8 else np.float16)
    a = orc.c_dequant(w.q, w.scale, w.zp, group)
    b = orc.np_dequant(w.q, w.scale, w.zp, group)
    np.testing.assert_array_equal(a, b)      # same fp32 steps -> same bits


def test_linear_c_vs_float64():
    x, w = synth.u4g128(4, 3, 48, 512)
    y = orc.linear(x, w.q, w.scale, w.zp, 128, out_dtype=np.float32)
    wdq = orc.np_dequant(w.q, w.scale, w.zp, 128)
    r = orc.np_dot_f64(x.astype(np.float32), wdq)
    assert orc.max_rel_err(y, r) < 2e-6
    y2 = orc.linear(x, w.q, w.scale, w.zp, 128, out_dtype=np.float32, naive_dot=True)
    assert orc.max_rel_err(y2, r) < 2e-6


def test_linear_prologue_epilogue_against_numpy():
    x, w = synth.u4g128(5, 2, 32, 256)
    rng = np.random.Generator(np.random.PCG64(6))
    w2 = synth.make_weights(rng, 32, 256, 4, 128)
    gain = rng.uniform(0.9, 1.1, 256).astype(np.float32)
    bias = rng.standard_normal(32).astype(np.float32)
    y = orc.linear(x, w.q, w.scale, w.zp, 128, q2=w2.q, scale2=w2.scale, zp2=w2.zp, gain=gain,
                   eps=1e-6, bias=bias, out_dtype=np.float32)
    xn = orc.np_rmsnorm(x.astype(np.float32), gain, 1e-6)
    g = orc.np_dot_f64(xn, orc.np_dequant(w.q, w.scale, w.zp, 128))
    u = orc.np_dot_f64(xn, orc.np_dequant(w2.q, w2.scale, w2.zp, 128))
    r = g / (1 + np.exp(-g)) * u + bias[None, :]
    assert orc.max_rel_err(y, r) < 5e-6


@needs_ref
def test_restated_sgemm_vs_reference_mlas():
    rng = np.random.default_rng(7)
    for (M, N, K) in [(1, 64, 256), (16, 96, 1024), (33, 130, 300), (5, 7, 129)]:
        a = rng.standard_normal((M, K)).astype(np.float32)
        b = rng.standard_normal((N, K)).astype(np.float32)
        r = orc.ref_sgemm(a, b, trans_b=True)
        y = orc.c_dot(a, b, trans_b=True, naive=False)
        assert orc.max_rel_err(y, r) < 2e-6, (M, N, K)
        assert orc.max_rel_err(r, orc.np_dot_f64(a, b)) < 2e-6


@needs_ref
def test_reference_graph_vs_oracle_config1_small():
    x, w = synth.config1(seed=0, M=16, N=256, K=512)
    graph = orc.RefLinearGraph(256, 512)
    r = graph(x, w.q, w.scale, w.zp, 512)
    np.testing.assert_array_equal(graph.wdq, orc.c_dequant(w.q, w.scale, w.zp, 512))
    y = orc.linear(x, w.q, w.scale, w.zp, 512)
    assert orc.max_rel_err(y, r) < 2e-6


def test_oracle_against_committed_mlas_fixture():
    """Outputs of the reference's MLAS path, generated by tests/golden/make_golden.py and committed."""
    import os
    from tests.golden import make_golden as mg
    fx = np.load(os.path.join(os.path.dirname(mg.__file__), "mlas_linear_small.npz"))
    for name, (kind, kw) in mg.CASES.items():
        x, w = mg.inputs(kind, kw)
        y = orc.linear(x.astype(np.float32), w.q, w.scale, w.zp, w.group, out_dtype=np.float32)
        assert orc.max_rel_err(y, fx[name]) < 2e-6, name
        y2 = orc.linear(x.astype(np.float32), w.q, w.scale, w.zp, w.group, out_dtype=np.float32, naive_dot=True)
        assert orc.max_rel_err(y2, fx[name]) < 2e-6, name
