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


@pytest.mark.parametrize("M", [32, 300])
def test_fp32_activations_through_the_prepass(M):
    """fp32 x (and fp32 y): a pre-pass rounds the activations to fp16 once, then the tensor-core kernel runs.  The
    fp32 path's tolerance of 1e-3 still holds (one rounding of x and one of the scale to fp16: a few 1e-4)."""
    x, w = synth.u4g128(35 + M, M, 136, 1024, x_dtype=np.float32)
    y = gpu_linear(x, w, kernel=L.KERNEL_GEMM)
    assert y.dtype == np.float32
    err = orc.max_rel_err(y, oracle_linear(x, w))
    assert err <= 1e-3, err


@pytest.mark.parametrize("M", [64, 256])
def test_config1_format_large_m(M):
    """Configuration 1's operand types (x fp32, uint8 weights, fp32 per-channel scale) at M above the small-M kernel's
    range, through automatic dispatch."""
    rng = np.random.Generator(np.random.PCG64(36))
    x = synth.make_x(rng, M, 4096, np.float32)
    w = synth.make_weights(rng, 512, 4096, 8, 4096, np.float32, (0.001, 0.01), (120, 137))
    y = gpu_linear(x, w)
    err = orc.max_rel_err(y, oracle_linear(x, w))
    assert err <= 1e-3, err


@pytest.mark.parametrize("xdt", [np.float16, np.float32])
@pytest.mark.parametrize("M,dual", [(40, False), (130, True)])
def test_rmsnorm_prologue_through_the_prepass(M, dual, xdt):
    rng = np.random.Generator(np.random.PCG64(37))
    K, N = 1024, 264
    x = synth.make_x(rng, M, K, xdt)
    gain = rng.uniform(0.9, 1.1, K).astype(np.float32)
    wg = synth.make_weights(rng, N, K, 4, 128)
    wu = synth.make_weights(rng, N, K, 4, 128) if dual else None
    y = gpu_linear(x, wg, wu, gain=gain, kernel=L.KERNEL_GEMM)
    _check(y, oracle_linear(x, wg, wu, gain=gain), TOL_F16, tight=3e-3)


def test_prepass_needs_its_workspace():
    import ctypes
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight
    x, w = synth.u4g128(38, 32, 128, 256, x_dtype=np.float32)
    op = DequantDot(DeviceWeight.from_host(w), kernel=L.KERNEL_GEMM)
    tx = torch.from_numpy(x).cuda()
    d = op.desc(32, tx.dtype)
    assert int(op.ctx.lib.nnf_b200_linear_workspace_bytes(op.ctx.handle, ctypes.byref(d))) >= 32 * 256 * 2
    y = torch.empty((32, 128), dtype=torch.float32, device="cuda")
    rc = op.ctx.lib.nnf_b200_linear(op.ctx.handle, torch.cuda.current_stream().cuda_stream, ctypes.byref(d),
                                    tx.data_ptr(), ctypes.byref(op._abi_w), None, None, None, y.data_ptr(), None, 0)
    assert rc == L.EWORKSPACE


# ---------------------------------------------------------------------------------------------------------------
# Persistent CTAs that share tiles: the work of a launch is cut evenly into raw-chunk units, so tiles at the seams
# are computed by two or more CTAs and added in a fixed order by the last one to arrive.

@pytest.mark.parametrize("M,N,K,bits", [
    (256, 1024, 4096, 4),     # 8 tiles of 16 chunks on 128 CTAs: every tile is shared by 16 CTAs
    (300, 2000, 2048, 4),     # ragged M and N, 32 tiles of 8 chunks: seams inside most tiles
    (520, 1280, 1024, 8),     # uint8 weights (two k-blocks per chunk)
    (64, 128, 320, 4),        # K / 64 = 5: the tile's last chunk holds one k-block, which only one group converts
    (96, 256, 192, 8),        # the same for uint8: three k-blocks, two per chunk
    (40, 128, 64, 4),         # a single k-block
])
def test_shared_tiles(M, N, K, bits):
    rng = np.random.Generator(np.random.PCG64(41 + M))
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, bits, 64 if K % 128 else 128)
    _check(gpu_linear(x, w, kernel=L.KERNEL_GEMM), oracle_linear(x, w), TOL_F16, tight=2e-3)


def test_shared_tiles_silu_mul_and_bias():
    rng = np.random.Generator(np.random.PCG64(42))
    M, N, K = 200, 1100, 2048
    x = synth.make_x(rng, M, K, np.float16)
    wg = synth.make_weights(rng, N, K, 4, 128)
    wu = synth.make_weights(rng, N, K, 4, 128)
    _check(gpu_linear(x, wg, wu, kernel=L.KERNEL_GEMM), oracle_linear(x, wg, wu), TOL_F16, tight=3e-3)
    bias = rng.standard_normal(N).astype(np.float32)
    _check(gpu_linear(x, wg, bias=bias, kernel=L.KERNEL_GEMM), oracle_linear(x, wg, bias=bias), TOL_F16, tight=2e-3)


def test_repeated_calls_share_one_workspace_and_agree_bitwise():
    """The arrival counters are left zeroed by every launch, and the order in which shared tiles are added does not
    depend on which CTA arrives last: the same call twice on one workspace gives the same bits."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight
    x, w = synth.u4g128(43, 256, 1024, 4096)
    op = DequantDot(DeviceWeight.from_host(w), kernel=L.KERNEL_GEMM)
    tx = torch.from_numpy(x).cuda()
    y0 = op(tx).clone()
    for _ in range(5):
        y1 = op(tx)
        assert torch.equal(y0, y1)
    op.ctx.device_status()


def test_shared_tiles_odd_n_scalar_stores():
    """N not a multiple of four: the CTA that adds a shared tile's slots stores element by element."""
    rng = np.random.Generator(np.random.PCG64(44))
    M, N, K = 300, 1001, 2048
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    _check(gpu_linear(x, w, kernel=L.KERNEL_GEMM), oracle_linear(x, w), TOL_F16, tight=2e-3)
    _check(gpu_linear(x, w, kernel=L.KERNEL_GEMM, out_dtype=np.float32), oracle_linear(x, w, out_dtype=np.float32),
           TOL_F16, tight=2e-3)


@pytest.mark.parametrize("N", [1024, 1001])
def test_shared_tiles_add_epilogue_in_place(N):
    """The full-size addend (also when it is y itself) through whole and shared tiles."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight
    rng = np.random.Generator(np.random.PCG64(45))
    M, K = 270, 2048
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    c = rng.standard_normal((M, N)).astype(np.float16)
    ref = (oracle_linear(x, w, out_dtype=np.float32).astype(np.float32) + c.astype(np.float32)).astype(np.float16)
    op = DequantDot(DeviceWeight.from_host(w, "cuda:0"), add=True, kernel=L.KERNEL_GEMM)
    tx, tc = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    y = op(tx, addend=tc)
    torch.cuda.synchronize()
    _check(y.cpu().numpy(), ref, TOL_F16, tight=2e-3)
    y2 = op(tx, out=tc, addend=tc)           # in place
    torch.cuda.synchronize()
    np.testing.assert_array_equal(y2.cpu().numpy(), y.cpu().numpy())
    op.ctx.device_status()


def test_silu_mul_fp32_output_and_odd_n():
    """SiLU(gate) * up as two launches that meet in y: fp32 y keeps the gate products in fp32; odd N takes the scalar
    path of the CTA that adds a shared tile's slots."""
    rng = np.random.Generator(np.random.PCG64(46))
    M, N, K = 130, 1001, 2048
    x = synth.make_x(rng, M, K, np.float16)
    wg = synth.make_weights(rng, N, K, 4, 128)
    wu = synth.make_weights(rng, N, K, 4, 128)
    _check(gpu_linear(x, wg, wu, kernel=L.KERNEL_GEMM), oracle_linear(x, wg, wu), TOL_F16, tight=3e-3)
    _check(gpu_linear(x, wg, wu, kernel=L.KERNEL_GEMM, out_dtype=np.float32),
           oracle_linear(x, wg, wu, out_dtype=np.float32), TOL_F16, tight=3e-3)


def test_output_padding_untouched_with_shared_tiles():
    """NaN-filled guard rows around y stay NaN when tiles are shared and M, N are ragged."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight
    x, w = synth.u4g128(47, 300, 1000, 2048)
    op = DequantDot(DeviceWeight.from_host(w, "cuda:0"), kernel=L.KERNEL_GEMM)
    tx = torch.from_numpy(x).cuda()
    guard = 64
    buf = torch.full((guard + 300 * 1000 + guard,), float("nan"), dtype=torch.float16, device="cuda")
    y = buf[guard:guard + 300 * 1000].view(300, 1000)
    op(tx, out=y)
    torch.cuda.synchronize()
    assert torch.isnan(buf[:guard]).all() and torch.isnan(buf[-guard:]).all()
    assert not torch.isnan(y).any()
    _check(y.cpu().numpy(), oracle_linear(x, w), TOL_F16, tight=2e-3)
    op.ctx.device_status()


@pytest.mark.parametrize("M,N,K,dual,launches", [
    (4096, 11008, 4096, False, 60),     # 9 tiles per CTA
    (256, 3584, 8192, True, 300),       # every tile shared by 6 CTAs, segments as short as one chunk, two passes
])
def test_back_to_back_launches_repeat_bit_for_bit(M, N, K, dual, launches):
    """Many launches in a row, no host synchronisation in between, must all give the first launch's bits.  Two races
    showed up only this way, as a few weight rows of one tile wrong for every batch row in a few launches per hundred:
    lanes that had left a polling loop on different rounds issued a warp-wide tensor-memory store apart, and a raw
    weight stage was handed back to the copy engine before the shared-memory loads from it had delivered."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    rng = np.random.Generator(np.random.PCG64(5 + M))
    dev = "cuda:0"
    ws = [DeviceWeight.from_host(synth.make_weights(rng, N, K, 4, 128), dev) for _ in range(2 if dual else 1)]
    op = DequantDot(*ws)
    x = torch.from_numpy(synth.make_x(rng, M, K, np.float16)).to(dev)
    first = op(x).clone()
    outs = [op(x) for _ in range(launches)]
    torch.cuda.synchronize()
    differ = [i for i, y in enumerate(outs) if not torch.equal(y, first)]
    op.ctx.device_status()
    assert not differ, f"launches {differ[:8]} of {launches} differ from the first"


@pytest.mark.parametrize("M", [17, 48, 64, 65])
@pytest.mark.parametrize("N,K,bits,dual", [
    (1024, 4096, 4, False),    # 8 tiles of 16 chunks on 128 CTAs: every tile shared by 16 CTAs
    (1001, 2048, 4, True),     # odd N (scalar stores), SiLU(gate) * up in two passes
    (640, 1024, 8, False),     # uint8 weights
])
def test_narrow_batch_tile(M, N, K, bits, dual):
    """Up to 64 batch rows the tensor-core kernel works on tiles of 64 batch rows (a quarter of the accumulator, of
    the activation tile and of a shared tile's slot); 65 rows are the first to take the 256-row tile again.  Both
    against the oracle, and three calls in a row bit for bit."""
    rng = np.random.Generator(np.random.PCG64(300 + M + N))
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, bits, 128)
    w2 = synth.make_weights(rng, N, K, bits, 128) if dual else None
    ys = gpu_linear(x, w, w2, kernel=L.KERNEL_GEMM, repeat=3)
    _check(ys[0], oracle_linear(x, w, w2), TOL_F16, tight=3e-3)
    assert all(np.array_equal(ys[0], y) for y in ys[1:])


def test_narrow_batch_tile_epilogues_and_padding():
    rng = np.random.Generator(np.random.PCG64(333))
    M, N, K = 40, 520, 2048
    x = synth.make_x(rng, M, K, np.float32)
    w = synth.make_weights(rng, N, K, 4, 128)
    bias = rng.standard_normal(N).astype(np.float32)
    gain = rng.uniform(0.5, 1.5, K).astype(np.float32)
    # fp32 activations and RMSNorm through the pre-pass, bias, fp32 output
    y = gpu_linear(x, w, gain=gain, bias=bias, kernel=L.KERNEL_GEMM, out_dtype=np.float32)
    _check(y, oracle_linear(x, w, gain=gain, bias=bias, out_dtype=np.float32), TOL_F16, tight=2e-3)
