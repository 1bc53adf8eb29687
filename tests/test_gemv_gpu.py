"""Parity of the small-M (decode) kernel with the CPU oracle, through the C-ABI, on a B200."""
import ctypes

import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import synth
from oracle import oracle as orc
from tests.util import TOL_F16, TOL_F32, gpu_linear, oracle_linear

pytestmark = pytest.mark.gpu


def _check(y, r, tol, tight=None):
    assert y.shape == r.shape and y.dtype == r.dtype
    err = orc.max_rel_err(y, r)
    assert err <= tol, f"max rel err {err:.3e} > {tol}"
    if tight is not None:
        assert err <= tight, f"max rel err {err:.3e} > expected {tight}"


@pytest.mark.parametrize("M", [1, 2, 3, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 128), (48, 256), (50, 384), (272, 4096)])
def test_u4_g128_fp16_small(M, N, K):
    x, w = synth.u4g128(100 + M, M, N, K)
    _check(gpu_linear(x, w), oracle_linear(x, w), TOL_F16, tight=1.5e-3)


@pytest.mark.parametrize("exact", [0, 1])
@pytest.mark.parametrize("M,N,K,bits", [(1, 64, 1024, 4), (7, 96, 2304, 4), (16, 48, 512, 4), (3, 80, 640, 8), (16, 32, 1024, 8)])
def test_exact_zero_point_flag(exact, M, N, K, bits):
    """Both zero-point treatments (removed before the multiply / taken out of the fp32 sum) meet the tolerance,
    and agree with each other to fp32 rounding."""
    from nnfusion_b200 import _lib as L
    rng = np.random.Generator(np.random.PCG64(77))
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, bits, 128)
    r = oracle_linear(x, w, out_dtype=np.float32)
    y = gpu_linear(x, w, out_dtype=np.float32, flags=L.FLAG_EXACT_ZP if exact else 0)
    _check(y, r, TOL_F16, tight=3e-5 if exact else 1e-4)


@pytest.mark.parametrize("N,K", [(11008, 4096), (4096, 11008)])
def test_config2_decode_gemv_full_size(N, K):
    x, w = synth.u4g128(0, 1, N, K)
    y = gpu_linear(x, w)
    r = oracle_linear(x, w)
    _check(y, r, TOL_F16, tight=1.5e-3)
    # linearity in x (size-independent property): f(2x) == 2 f(x) exactly in fp16 away from overflow
    y2 = gpu_linear((2 * x.astype(np.float32)).astype(np.float16), w)
    np.testing.assert_array_equal(y2.astype(np.float32), 2 * y.astype(np.float32))


def test_config1_u8_per_channel_fp32_full_size():
    x, w = synth.config1(0)
    y = gpu_linear(x, w)
    r = oracle_linear(x, w)
    _check(y, r, TOL_F32, tight=2e-5)
    if orc.have_ref():   # the reference's own MLAS behind its element-wise kernels
        rr = orc.RefLinearGraph(w.N, w.K)(x, w.q, w.scale, w.zp, w.group)
        _check(y, rr, TOL_F32, tight=2e-5)


@pytest.mark.parametrize("M", [1, 5, 16])
@pytest.mark.parametrize("group", [64, 128, 0])
def test_u8_groups_fp32(M, group):
    rng = np.random.Generator(np.random.PCG64(7))
    K, N = 512, 80
    x = synth.make_x(rng, M, K, np.float32)
    w = synth.make_weights(rng, N, K, 8, group or K, np.float32, (0.001, 0.01), (120, 136))
    _check(gpu_linear(x, w), oracle_linear(x, w), TOL_F32, tight=2e-5)


@pytest.mark.parametrize("M", [1, 4, 12])
def test_u8_fp16_activations(M):
    rng = np.random.Generator(np.random.PCG64(8))
    x = synth.make_x(rng, M, 1024, np.float16)
    w = synth.make_weights(rng, 96, 1024, 8, 128, np.float16, (0.001, 0.01))
    _check(gpu_linear(x, w), oracle_linear(x, w), TOL_F16, tight=1.5e-3)


@pytest.mark.parametrize("M", [1, 6, 16])
def test_u4_fp32_activations_fp32_scale(M):
    rng = np.random.Generator(np.random.PCG64(9))
    x = synth.make_x(rng, M, 768, np.float32)
    w = synth.make_weights(rng, 64, 768, 4, 128, np.float32, (0.002, 0.02))
    _check(gpu_linear(x, w), oracle_linear(x, w), TOL_F32, tight=None if M > 8 else 1e-4)


@pytest.mark.parametrize("M", [1, 8, 13])
def test_rmsnorm_prologue(M):
    rng = np.random.Generator(np.random.PCG64(10))
    x = synth.make_x(rng, M, 4096, np.float16)
    w = synth.make_weights(rng, 160, 4096, 4, 128)
    gain = rng.uniform(0.9, 1.1, 4096).astype(np.float32)
    _check(gpu_linear(x, w, gain=gain), oracle_linear(x, w, gain=gain), TOL_F16, tight=2e-3)


@pytest.mark.parametrize("M", [1, 3, 16])
def test_silu_mul_epilogue_with_rmsnorm(M):
    rng = np.random.Generator(np.random.PCG64(11))
    x = synth.make_x(rng, M, 2048, np.float16)
    wg = synth.make_weights(rng, 176, 2048, 4, 128)
    wu = synth.make_weights(rng, 176, 2048, 4, 128)
    gain = rng.uniform(0.9, 1.1, 2048).astype(np.float32)
    _check(gpu_linear(x, wg, wu, gain=gain), oracle_linear(x, wg, wu, gain=gain), TOL_F16, tight=2e-3)


@pytest.mark.parametrize("M", [1, 16])
def test_bias_epilogue(M):
    rng = np.random.Generator(np.random.PCG64(12))
    x = synth.make_x(rng, M, 512, np.float16)
    w = synth.make_weights(rng, 40, 512, 4, 128)
    bias = rng.standard_normal(40).astype(np.float32)
    _check(gpu_linear(x, w, bias=bias), oracle_linear(x, w, bias=bias), TOL_F16, tight=1.5e-3)


@pytest.mark.parametrize("split_k", [3, 4, 7, 43])
def test_split_k_agrees_and_workspace_is_reusable(split_k):
    x, w = synth.u4g128(13, 2, 200, 11008)
    r = oracle_linear(x, w)
    ys = gpu_linear(x, w, split_k=split_k, repeat=3)   # same workspace, three calls in a row
    for y in ys:
        _check(y, r, TOL_F16, tight=1.5e-3)
    np.testing.assert_array_equal(ys[0], ys[1])         # fixed summation order: bitwise repeatable
    np.testing.assert_array_equal(ys[0], ys[2])


def test_split_k_too_small_is_rejected():
    """One CTA has at most 16 warps, one per 128-byte slice of a row: K = 8192 (32 slices) needs two splits."""
    x, w = synth.u4g128(13, 1, 16, 8192)
    with pytest.raises(RuntimeError, match="split_k too small"):
        gpu_linear(x, w, split_k=1)
    assert len(gpu_linear(x, w, split_k=2, repeat=2)) == 2
    _check(gpu_linear(x, w), oracle_linear(x, w), TOL_F16, tight=1.5e-3)


def test_empty_and_invalid_arguments():
    import torch
    from nnfusion_b200 import _lib as L
    from nnfusion_b200.linear import DequantDot, DeviceWeight, NNFB200Error

    x, w = synth.u4g128(14, 1, 32, 256)
    dw = DeviceWeight.from_host(w)
    op = DequantDot(dw)
    tx = torch.from_numpy(x).cuda()
    # M = 0 is rejected by the descriptor check (the reference's Dot also refuses empty operands at
    # code generation: src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:44-85 handles only scalars).
    d = op.desc(1, tx.dtype)
    d.M = 0
    with pytest.raises(NNFB200Error) as e:
        op.run_raw(d, tx.data_ptr(), tx.data_ptr(), None)
    assert e.value.status == L.EINVAL
    # K not a multiple of the 64-byte unit
    d = op.desc(1, tx.dtype)
    d.K = 192
    with pytest.raises(NNFB200Error) as e:
        op.run_raw(d, tx.data_ptr(), tx.data_ptr(), None)
    assert e.value.status == L.ENOTSUP
    # misaligned activations
    d = op.desc(1, tx.dtype)
    with pytest.raises(NNFB200Error) as e:
        op.run_raw(d, tx.data_ptr() + 2, tx.data_ptr(), None)
    assert e.value.status == L.EALIGN
    # split-K without a workspace
    xb, wb = synth.u4g128(15, 1, 32, 11008)
    opb = DequantDot(DeviceWeight.from_host(wb), split_k=4)
    txb = torch.from_numpy(xb).cuda()
    d = opb.desc(1, txb.dtype)
    y = torch.empty((1, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(NNFB200Error) as e:
        opb.run_raw(d, txb.data_ptr(), y.data_ptr(), None)
    assert e.value.status == L.EWORKSPACE
    # gain without the prologue
    with pytest.raises(NNFB200Error) as e:
        opb.ctx.check(opb.ctx.lib.nnf_b200_linear(opb.ctx.handle, None, ctypes.byref(d), txb.data_ptr(),
                                                  ctypes.byref(opb._abi_w), None, txb.data_ptr(), None,
                                                  y.data_ptr(), None, 0))
    assert e.value.status == L.EINVAL


def test_output_padding_untouched():
    """Ragged N (not a multiple of the 16-row tile): nothing is written past the last column."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    x, w = synth.u4g128(16, 3, 50, 256)
    op = DequantDot(DeviceWeight.from_host(w))
    tx = torch.from_numpy(x).cuda()
    big = torch.full((3 * 50 + 64,), float("nan"), dtype=torch.float16, device="cuda")
    d = op.desc(3, tx.dtype)
    op.run_raw(d, tx.data_ptr(), big.data_ptr(), op.workspace(d))
    torch.cuda.synchronize()
    out = big.cpu().numpy()
    assert np.isnan(out[150:]).all()
    _check(out[:150].reshape(3, 50), oracle_linear(x, w), TOL_F16, tight=1.5e-3)


@pytest.mark.parametrize("K", [2304, 4480, 7168, 11008])
@pytest.mark.parametrize("M,N,bits,group,xdt,dual", [
    (1, 4096, 4, 128, np.float16, False), (1, 1008, 4, 128, np.float16, True),
    (3, 272, 8, 64, np.float32, False), (16, 1024, 4, 128, np.float16, False)])
def test_k_split_with_idle_warps_after_other_kernels_used_shared_memory(K, M, N, bits, group, xdt, dual):
    """K values whose 128-byte slices do not divide evenly over the CTAs that share a row: some warps have no slice,
    and CTAs copy only their own columns of the scales and zero-points.  A large-M call first leaves arbitrary bit
    patterns in shared memory, so a warp that multiplied zero activations with parameters nobody copied would show."""
    rng = np.random.Generator(np.random.PCG64(500 + K + M))
    xg = (rng.standard_normal((64, 256)) * 1e4).astype(np.float16)
    gpu_linear(xg, synth.make_weights(rng, 256, 256, 8, 64), kernel=L.KERNEL_GEMM)
    x = synth.make_x(rng, M, K, xdt)
    sd = np.float32 if xdt == np.float32 else np.float16
    w = synth.make_weights(rng, N, K, bits, group, sd)
    w2 = synth.make_weights(rng, N, K, bits, group, sd) if dual else None
    _check(gpu_linear(x, w, w2), oracle_linear(x, w, w2), TOL_F32 if xdt == np.float32 else TOL_F16)


@pytest.mark.parametrize("M,N,K,split_k,dual,norm", [
    (1, 33 * 74 * 16, 8192, 0, False, False),   # halves of K as clusters of 2; 33 tiles per CTA: two batches
    (3, 2048, 8192, 0, True, True),             # RMSNorm + SiLU(gate) * up: sums of squares meet in shared memory too
    (2, 208, 4096, 4, False, False),            # 13 tiles: 13 clusters of 4 fit at once
    (1, 160, 7168, 7, False, True),             # 10 clusters of 7
    (5, 1024, 2048, 8, False, False),           # one slice per CTA, clusters of 8 (the device holds 15 at most: workspace)
])
def test_k_splits_that_meet_in_shared_memory(M, N, K, split_k, dual, norm):
    """K splits whose CTAs form a thread-block cluster add their sums in the first CTA's shared memory; the same
    descriptor falls back to the workspace when the device cannot hold every cluster at once.  Either way the result
    matches the oracle and repeats bit for bit."""
    rng = np.random.Generator(np.random.PCG64(77 + N))
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    w2 = synth.make_weights(rng, N, K, 4, 128) if dual else None
    gain = rng.uniform(0.5, 1.5, K).astype(np.float32) if norm else None
    ys = gpu_linear(x, w, w2, gain=gain, split_k=split_k, repeat=3)
    ref = oracle_linear(x, w, w2, gain=gain)
    assert orc.max_rel_err(ys[0], ref) <= TOL_F16
    assert all(np.array_equal(ys[0], y) for y in ys[1:])
