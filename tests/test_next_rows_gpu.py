"""GPU tests of the pieces around the kernels: constants uploaded from disk, the front-door module, and launch
choices taken from the kernel database."""
import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import constants, kernel_db, synth
from oracle import oracle as orc
from tests.util import TOL_F16, oracle_linear

pytestmark = pytest.mark.gpu


def test_constants_from_disk_run_unchanged(tmp_path):
    import torch
    from nnfusion_b200.linear import DequantDot

    x, w = synth.u4g128(21, 3, 272, 1024)
    constants.save_linear(str(tmp_path), "blk.ffn_up", w)
    dw = constants.load_linear(str(tmp_path), "blk.ffn_up", "cuda:0")
    assert torch.equal(dw.wq.cpu(), torch.from_numpy(w.wq))       # the bytes on disk are the bytes in HBM
    y = DequantDot(dw)(torch.from_numpy(x).cuda()).cpu().numpy()
    assert orc.max_rel_err(y, oracle_linear(x, w)) <= TOL_F16


@pytest.mark.parametrize("via_onnx", [False, True])
@pytest.mark.parametrize("M", [1, 33])
def test_front_door_allclose(M, via_onnx, tmp_path):
    # shaped like the reference's test/python/test_jit.py:8-40: the wrapped module against plain PyTorch
    import torch
    from nnfusion_b200.jit import QuantLinear, jit

    rng = np.random.Generator(np.random.PCG64(31))
    w1, w2 = synth.make_weights(rng, 512, 256, 4, 128), synth.make_weights(rng, 128, 512, 4, 128)
    bias = rng.standard_normal(128).astype(np.float32)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2 = QuantLinear.from_host(w1), QuantLinear.from_host(w2, bias)

        def forward(self, x):
            return self.fc2(torch.relu(self.fc1(x)))

    # via_onnx: every quantised linear goes module -> ONNX file (Cast / Sub / Mul / Gemm) -> fold -> fused node
    net = jit(Net().cuda(), onnx_dir=str(tmp_path) if via_onnx else None)
    if via_onnx:
        import os
        from nnfusion_b200 import onnx_writer
        assert sorted(os.listdir(tmp_path)) == ["fc1.onnx", "fc2.onnx"]
        ops = [n["op_type"] for n in onnx_writer.read_model(str(tmp_path / "fc2.onnx"))["graph"]["nodes"]]
        assert ops == ["Reshape", "Cast", "Cast", "Sub", "Mul", "Reshape", "Gemm"]
        np.testing.assert_array_equal(net.fc1.wq.cpu().numpy(), w1.wq)      # the same packed bytes come back
    x = torch.from_numpy(synth.make_x(rng, M, 256, np.float16)).cuda().reshape(M, 1, 256)
    y = net(x)
    assert y.shape == (M, 1, 128) and y.dtype == torch.float16
    h = torch.relu(x.float() @ net.fc1.dequantized().T).half().float()
    ref = h @ net.fc2.dequantized().T + net.fc2.bias
    torch.testing.assert_close(y.float(), ref, rtol=5e-3, atol=5e-3 * float(ref.abs().max()))


def test_launch_choice_from_the_database(tmp_path):
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    x, w = synth.u4g128(41, 4, 256, 2048)
    dw = DeviceWeight.from_host(w, "cuda:0")
    tx = torch.from_numpy(x).cuda()
    db = kernel_db.KernelCacheManager(str(tmp_path / "kernel_cache.db"))
    ident = kernel_db.identifier(4, 256, 2048, 4, 128, L.F16, L.F16, L.F16)
    measure = kernel_db.measure_on_gpu(lambda fn: DequantDot(dw, kernel=fn["kernel"], split_k=fn["split_k"]), tx, 20)
    best = kernel_db.tune(db, ident, kernel_db.default_candidates(4), measure, "B200")
    assert best is not None and best.time_us("B200") > 0
    stored = db.fetch_all(ident)
    assert len(stored) >= 3                                       # refused combinations are simply absent
    # a node that consults the database runs what the database says, and computes the same thing
    op = DequantDot(dw, kernel_db=db)
    d = op.desc(4, torch.float16)
    assert (d.kernel, d.split_k) == (best.function["kernel"], best.function["split_k"])
    y = op(tx).cpu().numpy()
    assert orc.max_rel_err(y, oracle_linear(x, w)) <= TOL_F16
    # other shapes fall back to the built-in rule
    assert DequantDot(dw, kernel_db=db).desc(5, torch.float16).kernel == L.KERNEL_AUTO


def test_host_entry_copies_in_and_out():
    # the host-buffer entry point (kernel_entry_host of the generated runtime): pinned x in, pinned y out
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    x, w = synth.u4g128(51, 2, 272, 1024)
    op = DequantDot(DeviceWeight.from_host(w, "cuda:0"))
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.empty((2, 272), dtype=torch.float16).pin_memory()
    op.host_entry(xh, yh)
    ref = oracle_linear(x, w)
    assert orc.max_rel_err(yh.numpy(), ref) <= TOL_F16
    xh.mul_(2)                                   # new contents, same buffers: the captured graph is reused
    op.host_entry(xh, yh)
    assert orc.max_rel_err(yh.numpy(), oracle_linear(xh.numpy(), w)) <= TOL_F16
    with pytest.raises(ValueError):
        op.host_entry(torch.from_numpy(x), yh)   # not pinned
