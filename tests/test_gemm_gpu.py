"""Parity of the large-M (prefill) tcgen05 kernel with the CPU oracle, through the C-ABI, on a B200."""
import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import synth
from oracle import oracle as orc
from tests.util import TOL_F16, gpu_linear, oracle_linear

pytestmark = pytest.mark.gpu


def _check(y, r, tol, tight=None):
    assert y.shape == r.shape and y.dtype == r.dtype
    err = orc.max_rel_err(y, r)
    assert err <= tol, f"max rel err {err:.3e} > {tol}"
    if tight is not None:
        assert err <= tight, f"max rel err {err:.3e} > expected {tight}"


def test_single_tile_known_pattern():
    """One CTA, one k-chunk: weights q = column index mod 16 with zp = 0, scale = 1 and x = one-hot rows, so that
    y[m, n] = q[n, m]: any mistake in the k order of the tensor-memory operand shows up as a permutation."""
    M, N, K = 64, 128, 256
    q = (np.arange(K, dtype=np.uint8)[None, :] + np.arange(N, dtype=np.uint8)[:, None]) % 16
    w = synth.QuantLinear(N, K, 4, 128, q, np.ones((N, K // 128), np.float16), np.zeros((N, K // 128), np.uint8))
    x = np.zeros((M, K), np.float16)
    x[np.arange(M), np.arange(M) * 3 % K] = 1.0
    y = gpu_linear(x, w, kernel=L.KERNEL_GEMM, out_dtype=np.float32)
    want = q[:, np.arange(M) * 3 % K].T.astype(np.float32)
    np.testing.assert_array_equal(y, want)


@pytest.mark.parametrize("M,N,K", [(17, 128, 128), (256, 128, 256), (300, 200, 512), (64, 384, 1024), (513, 130, 4096)])
def test_u4_g128_small(M, N, K):
    x, w = synth.u4g128(200 + M, M, N, K)
    _check(gpu_linear(x, w, kernel=L.KERNEL_GEMM), oracle_linear(x, w), TOL_F16, tight=2e-3)


@pytest.mark.parametrize("M", [33, 256])
@pytest.mark.parametrize("group", [64, 128, 0])
def test_u8_groups(M, group):
    rng = np.random.Generator(np.random.PCG64(31))
    K, N = 512, 144
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 8, group or K, np.float16, (0.0005, 0.002), (120, 136))
    _check(gpu_linear(x, w, kernel=L.KERNEL_GEMM), oracle_linear(x, w), TOL_F16, tight=2e-3)


@pytest.mark.parametrize("M,N,K", [(40, 128, 256), (257, 300, 1024)])
def test_silu_mul_epilogue(M, N, K):
    rng = np.random.Generator(np.random.PCG64(32))
    x = synth.make_x(rng, M, K, np.float16)
    wg = synth.make_weights(rng, N, K, 4, 128)
    wu = synth.make_weights(rng, N, K, 4, 128)
    _check(gpu_linear(x, wg, wu, kernel=L.KERNEL_GEMM), oracle_linear(x, wg, wu), TOL_F16, tight=3e-3)


def test_bias_epilogue_fp32_output():
    rng = np.random.Generator(np.random.PCG64(33))
    x = synth.make_x(rng, 100, 512, np.float16)
    w = synth.make_weights(rng, 136, 512, 4, 128)
    bias = rng.standard_normal(136).astype(np.float32)
    _check(gpu_linear(x, w, bias=bias, kernel=L.KERNEL_GEMM, out_dtype=np.float32),
           oracle_linear(x, w, bias=bias, out_dtype=np.float32), TOL_F16, tight=2e-3)


def test_auto_dispatch_agrees_with_small_m_kernel():
    """M = 16 goes to the HBM-bound kernel, M = 17 to the tensor-core one: the shared rows agree within tolerance."""
    x, w = synth.u4g128(34, 17, 256, 1024)
    y17 = gpu_linear(x, w)
    y16 = gpu_linear(x[:16], w)
    assert orc.max_rel_err(y17[:16], y16) < 2e-3


@pytest.mark.parametrize("N,K", [(11008, 4096), (4096, 11008)])
def test_config3_prefill_m256_full_size(N, K):
    x, w = synth.u4g128(0, 256, N, K)
    y = gpu_linear(x, w)
    _check(y, oracle_linear(x, w), TOL_F16, tight=2e-3)


def test_unsupported_combinations_are_refused():
    from nnfusion_b200.linear import NNFB200Error
    x, w = synth.u4g128(35, 32, 128, 256, x_dtype=np.float32)
    with pytest.raises(NNFB200Error) as e:
        gpu_linear(x, w, kernel=L.KERNEL_GEMM)
    assert e.value.status == L.ENOTSUP
    x, w = synth.u4g128(36, 32, 128, 256)
    with pytest.raises(NNFB200Error) as e:
        gpu_linear(x, w, gain=np.ones(256, np.float32), kernel=L.KERNEL_GEMM)
    assert e.value.status == L.ENOTSUP
