"""The allocation-free entry point, for callers that can no longer ask CUDA for memory (a memory budget frozen
after start-up, a fixed GPU quota): it takes its split-K scratch from an array built into the
library instead of from a caller-provided workspace.  Its result must equal that of the regular entry point.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import synth

pytestmark = pytest.mark.gpu


def _static_call(lib, op, d, x, y):
    import torch
    err = ctypes.create_string_buffer(256)
    rc = lib.nnf_b200_linear_static_scratch(
        torch.cuda.current_stream().cuda_stream, ctypes.byref(d), x.data_ptr(), ctypes.byref(op._abi_w),
        ctypes.byref(op._abi_w2) if op._abi_w2 is not None else None,
        op.gain.data_ptr() if op.gain is not None else None, op.bias.data_ptr() if op.bias is not None else None,
        y.data_ptr(), err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("M,N,K,dual", [(1, 4096, 11008, False), (5, 528, 8192, True)])
def test_static_scratch_matches_regular_entry_point_twice_in_a_row(M, N, K, dual):
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    lib = L.load()
    rng = np.random.Generator(np.random.PCG64(91))
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    w2 = synth.make_weights(rng, N, K, 4, 128) if dual else None
    op = DequantDot(DeviceWeight.from_host(w), DeviceWeight.from_host(w2) if dual else None)
    tx = torch.from_numpy(x).cuda()
    d = op.desc(M, tx.dtype)
    plan = (ctypes.c_int32 * 8)()
    assert lib.nnf_b200_linear_plan(op.ctx.handle, ctypes.byref(d), ctypes.byref(plan)) == L.OK
    assert plan[2] > 1, "the case must exercise split-K, i.e. the scratch"
    want = op(tx)                                   # regular entry point, caller-provided workspace
    torch.cuda.synchronize()
    for call in range(2):                           # the array keeps the first call's contents for the second
        got = torch.full_like(want, float("nan"))
        rc, msg = _static_call(lib, op, d, tx, got)
        assert rc == L.OK, msg
        torch.cuda.synchronize()
        # same kernel, same launch shape, same fixed summation order: the tolerance of the fp16 path is met with
        # room to spare (the results are in fact bit-identical)
        a, b = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.max(np.abs(a - b)) <= 5e-3 * np.max(np.abs(b)), f"call {call}"
        np.testing.assert_array_equal(a, b)


def test_static_scratch_refuses_what_does_not_fit():
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    lib = L.load()
    # 16 batch rows x SiLU*mul: 528 floats per (split, tile) slot; 4096 tiles x 3 splits need 26 MB > 4 MiB
    N, K = 65536, 8192
    wq = torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda")
    sc = torch.ones((N, K // 128), dtype=torch.float16, device="cuda")
    zp = torch.zeros((N, K // 256), dtype=torch.uint8, device="cuda")
    dw = DeviceWeight(N, K, 4, 128, wq, sc, zp)
    op = DequantDot(dw, dw)
    x = torch.zeros((16, K), dtype=torch.float16, device="cuda")
    y = torch.zeros((16, N), dtype=torch.float16, device="cuda")
    rc, msg = _static_call(lib, op, op.desc(16, x.dtype), x, y)
    assert rc == L.EWORKSPACE
    assert str(L.STATIC_SCRATCH_BYTES) in msg and "scratch" in msg
    rc, msg = _static_call(lib, op, op.desc(17, x.dtype), x, y)      # M > 16 belongs to the other kernel
    assert rc == L.ENOTSUP


def test_static_scratch_survives_a_change_of_shape():
    """The built-in array keeps what the last call left.  A shape with few row tiles, then one with many (its tile
    counters and partial-sum slots spread over what the first one used, and beyond), then the first again: every
    result equals the regular entry point's, bit for bit, and no device-side wait has given up on the way."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    lib = L.load()
    rng = np.random.Generator(np.random.PCG64(92))
    cases = []
    for M, N, K in ((2, 272, 8192), (1, 4096, 11008), (3, 48, 16384)):
        w = synth.make_weights(rng, N, K, 4, 128)
        op = DequantDot(DeviceWeight.from_host(w))
        tx = torch.from_numpy(synth.make_x(rng, M, K, np.float16)).cuda()
        d = op.desc(M, tx.dtype)
        plan = (ctypes.c_int32 * 8)()
        assert lib.nnf_b200_linear_plan(op.ctx.handle, ctypes.byref(d), ctypes.byref(plan)) == L.OK
        assert plan[2] > 1, "every case must use the scratch"
        cases.append((op, tx, d, op(tx)))
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for i in (0, 1, 0, 2, 1, 2, 0):
        op, tx, d, want = cases[i]
        got = torch.full_like(want, float("nan"))
        rc, msg = _static_call(lib, op, d, tx, got)
        assert rc == L.OK, msg
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got.float().cpu().numpy(), want.float().cpu().numpy())
    assert lib.nnf_b200_static_scratch_status(stream) == L.OK


def test_static_scratch_checks_its_descriptor_like_the_regular_entry_point():
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    lib = L.load()
    rng = np.random.Generator(np.random.PCG64(93))
    w = synth.make_weights(rng, 64, 1024, 4, 128)
    op = DequantDot(DeviceWeight.from_host(w))
    x = torch.zeros((1, 1024), dtype=torch.float16, device="cuda")
    y = torch.zeros((1, 64), dtype=torch.float16, device="cuda")
    for field, value, status in (("x_dtype", 7, L.EINVAL), ("flags", 64, L.EINVAL), ("kernel", L.KERNEL_GEMM, L.ENOTSUP),
                                 ("epilogue", 9, L.EINVAL), ("prologue", 5, L.EINVAL)):
        d = op.desc(1, x.dtype)
        setattr(d, field, value)
        rc, msg = _static_call(lib, op, d, x, y)
        assert rc == status and msg, field
