"""A generated ``nnfusion_rt`` project, built with nvcc against ``libnnf_b200.so`` and opened the way the reference's
Python ``Executor`` opens one (``nnfusion_b200/runtime_loader.py``): ``get_device_type`` -> ``cuda_init`` (reads
``Constant/*.bin`` relative to the runtime directory) -> ``para_info.json`` -> ``kernel_entry_host`` / ``kernel_entry`` ->
``cuda_free``.  Results are compared with the CPU oracle."""
import ctypes

import numpy as np
import pytest

from nnfusion_b200 import codegen, runtime_loader, synth
from oracle import oracle as orc
from tests.util import TOL_F16, TOL_F32, oracle_linear

pytestmark = pytest.mark.gpu


def _project(tmp_path, node):
    out = str(tmp_path / "nnfusion_rt" / "cuda_codegen")
    codegen.generate(out, node)
    codegen.build(out)
    return out


def test_config1_graph_through_the_generated_runtime(tmp_path):
    """Configuration 1: X f32 [16,4096], W u8 [4096,4096], one fp32 scale and one u8 zero-point per output row."""
    rng = np.random.Generator(np.random.PCG64(0))
    x = synth.make_x(rng, 16, 4096, np.float32)
    w = synth.make_weights(rng, 4096, 4096, 8, 4096, np.float32, (0.001, 0.01), (120, 137))
    rt = _project(tmp_path, codegen.DequantDotNode("DequantDot_0", 16, w, x_dtype="float32"))
    ex = runtime_loader.RuntimeExecutor(rt)
    assert ex.host_entry and ex.device_type == 0
    assert [(i.name, i.dtype, i.shape) for i in ex.inputs] == [("x", "float32", (16, 4096))]
    assert [(o.name, o.dtype, o.shape) for o in ex.outputs] == [("y", "float32", (16, 4096))]
    y = np.full((16, 4096), np.nan, np.float32)
    for _ in range(2):
        assert ex({"x": runtime_loader.feed_numpy(x)}, {"y": runtime_loader.feed_numpy(y)}) == 0
    err = orc.max_rel_err(y, oracle_linear(x, w))
    assert err <= TOL_F32, err
    with pytest.raises(TypeError):
        ex({"x": runtime_loader.feed_numpy(x[:8])}, {"y": runtime_loader.feed_numpy(y)})
    with pytest.raises(KeyError):
        ex({"x": runtime_loader.feed_numpy(x), "z": runtime_loader.feed_numpy(x)}, {"y": runtime_loader.feed_numpy(y)})
    ex.close()


def test_uint4_linear_with_bias_device_entry(tmp_path):
    """A packed uint4 group-128 linear with a bias, fp16 in and out, fed with device tensors through kernel_entry."""
    import torch
    rng = np.random.Generator(np.random.PCG64(1))
    M, N, K = 1, 11008, 4096
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    bias = rng.standard_normal(N).astype(np.float32)
    rt = _project(tmp_path, codegen.DequantDotNode("DequantDot_0", M, w, epilogue="bias", bias=bias))
    ex = runtime_loader.RuntimeExecutor(rt)
    ex.entry = ex.lib.kernel_entry          # device pointers: the entry point without the copies
    tx = torch.from_numpy(x).cuda()
    ty = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    assert ex({"x": runtime_loader.feed_torch(tx)}, {"y": runtime_loader.feed_torch(ty)}) == 0
    torch.cuda.synchronize()
    err = orc.max_rel_err(ty.cpu().numpy(), oracle_linear(x, w, bias=bias))
    assert err <= TOL_F16, err
    ex.close()


def test_residual_add_epilogue_through_the_generated_runtime(tmp_path):
    """The add epilogue (MatMulAdd with its full-size addend) as the operator now expresses it."""
    rng = np.random.Generator(np.random.PCG64(2))
    M, N, K = 5, 512, 1024
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    c = rng.standard_normal((M, N)).astype(np.float16)
    rt = _project(tmp_path, codegen.DequantDotNode("DequantDot_0", M, w, epilogue="add"))
    ex = runtime_loader.RuntimeExecutor(rt)
    y = np.zeros((M, N), np.float16)
    assert ex({"x": runtime_loader.feed_numpy(x), "addend": runtime_loader.feed_numpy(c)},
              {"y": runtime_loader.feed_numpy(y)}) == 0
    want = (oracle_linear(x, w, out_dtype=np.float32) + c.astype(np.float32)).astype(np.float16)
    assert orc.max_rel_err(y, want) <= TOL_F16
    ex.close()


def test_host_entry_writes_into_pinned_result_buffers(tmp_path):
    """kernel_entry_host with a pinned result buffer: the node stores its result straight into host memory (no copy
    back); with a pageable one the result is copied.  Same bits either way, fresh inputs on every call."""
    import torch
    rng = np.random.Generator(np.random.PCG64(2))
    M, N, K = 1, 1024, 2048
    w = synth.make_weights(rng, N, K, 4, 128)
    rt = _project(tmp_path, codegen.DequantDotNode("DequantDot_0", M, w))
    ex = runtime_loader.RuntimeExecutor(rt)
    assert ex.host_entry
    xh = torch.empty((M, K), dtype=torch.float16).pin_memory()
    yh = torch.empty((M, N), dtype=torch.float16).pin_memory()
    for call in range(4):
        x = synth.make_x(rng, M, K, np.float16)
        xh.copy_(torch.from_numpy(x))
        yh.fill_(float("nan"))
        assert ex({"x": runtime_loader.feed_torch(xh)}, {"y": runtime_loader.feed_torch(yh)}) == 0
        err = orc.max_rel_err(yh.numpy().copy(), oracle_linear(x, w))
        assert err <= TOL_F16, (call, err)
    y2 = np.full((M, N), np.nan, np.float16)           # pageable: the copy path
    assert ex({"x": runtime_loader.feed_numpy(x)}, {"y": runtime_loader.feed_numpy(y2)}) == 0
    np.testing.assert_array_equal(y2, yh.numpy())
    ex.close()
