"""Full-size parity of the shapes whose throughput the benchmark quotes, and writes that must not stray.

* configuration 3 (prefill) at M = 1024 and 4096, both weight shapes: the GPU computes every row; a seeded sample of
  64 rows of x (every column of them) is compared with the oracle, whose rows do not depend on each other;
* configuration 5 (70B-shaped MLP): the unsharded linears and the two-rank shard shapes at M = 1 and 16, and one rank
  shard at M = 256 through the tensor-core kernel;
* uint8 weights with fp32 per-channel scales through the tensor-core kernel (the format of configuration 1);
* memory around the outputs filled with NaN beforehand stays NaN: the tensor-core kernel's stores for ragged M and N
  (fp16 and fp32 outputs), the attention kernel's cache rows past the new token.
"""
import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import synth
from nnfusion_b200.tp import mlp_shapes
from oracle import oracle as orc
from tests.util import TOL_F16, gpu_linear, oracle_linear

pytestmark = pytest.mark.gpu

SAMPLE_ROWS = 64


@pytest.mark.parametrize("M", [1024, 4096])
@pytest.mark.parametrize("N,K", [(11008, 4096), (4096, 11008)])
def test_config3_prefill_full_size_sampled_rows(M, N, K):
    x, w = synth.u4g128(3, M, N, K)
    y = gpu_linear(x, w)
    assert y.shape == (M, N) and y.dtype == np.float16 and np.isfinite(y.astype(np.float32)).all()
    rows = np.sort(np.random.Generator(np.random.PCG64(M + N)).choice(M, SAMPLE_ROWS, replace=False))
    rows[0], rows[-1] = 0, M - 1                      # the first and the last row are always in the sample
    r = oracle_linear(np.ascontiguousarray(x[rows]), w)
    err = orc.max_rel_err(y[rows], r)
    assert err <= TOL_F16, f"max rel err {err:.3e}"
    assert err <= 2e-3, f"max rel err {err:.3e} above what this kernel has shown so far"


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("M", [1, 16])
def test_mlp70b_unsharded_and_two_rank_shapes(world, M):
    (n_gu, k_gu), (n_d, k_d) = mlp_shapes(8192, 28672, world)
    rng = np.random.Generator(np.random.PCG64(900 + world))
    x = synth.make_x(rng, M, k_gu, np.float16)
    gate = synth.make_weights(rng, n_gu, k_gu, 4, 128)
    up = synth.make_weights(rng, n_gu, k_gu, 4, 128)
    h = gpu_linear(x, gate, up)
    assert orc.max_rel_err(h, oracle_linear(x, gate, up)) <= TOL_F16
    del gate, up
    down = synth.make_weights(rng, n_d, k_d, 4, 128)
    y = gpu_linear(h, down)
    assert y.shape == (M, n_d)
    assert orc.max_rel_err(y, oracle_linear(h, down)) <= TOL_F16


def test_mlp70b_rank_shard_m256_tensor_core_kernel():
    (n_gu, k_gu), (n_d, k_d) = mlp_shapes(8192, 28672, 8)
    rng = np.random.Generator(np.random.PCG64(908))
    x = synth.make_x(rng, 256, k_gu, np.float16)
    gate = synth.make_weights(rng, n_gu, k_gu, 4, 128)
    up = synth.make_weights(rng, n_gu, k_gu, 4, 128)
    h = gpu_linear(x, gate, up)
    assert orc.max_rel_err(h, oracle_linear(x, gate, up)) <= TOL_F16
    down = synth.make_weights(rng, n_d, k_d, 4, 128)
    assert orc.max_rel_err(gpu_linear(h, down), oracle_linear(h, down)) <= TOL_F16


@pytest.mark.parametrize("M", [64, 300])
def test_u8_fp32_per_channel_scales_through_the_tensor_core_kernel(M):
    """Configuration 1's weight format (uint8, one fp32 scale and one zero-point per output row) with fp16
    activations: the tensor-core kernel rounds the scale to fp16 before it multiplies, which must stay inside the
    fp16 path's tolerance."""
    rng = np.random.Generator(np.random.PCG64(41))
    N, K = 520, 4096
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 8, K, np.float32, (0.001, 0.01), (120, 136))
    y = gpu_linear(x, w, kernel=L.KERNEL_GEMM)
    assert orc.max_rel_err(y, oracle_linear(x, w)) <= TOL_F16


@pytest.mark.parametrize("M,N,out", [(130, 200, np.float16), (257, 136, np.float32), (17, 24, np.float16)])
def test_tensor_core_kernel_writes_nothing_outside_y(M, N, out):
    """Ragged M and N against the kernel's 128 x 256 tiles: y sits inside a larger NaN-filled buffer; the kernel must
    leave every byte in front of and behind it alone."""
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    K = 512
    x, w = synth.u4g128(77 + M, M, N, K)
    tdt = torch.float16 if out == np.float16 else torch.float32
    op = DequantDot(DeviceWeight.from_host(w), y_dtype=tdt, kernel=L.KERNEL_GEMM)
    tx = torch.from_numpy(x).cuda()
    pad = 4096                                          # elements of poison on either side (keeps y 16-byte aligned)
    big = torch.full((pad + M * N + pad,), float("nan"), dtype=tdt, device="cuda")
    d = op.desc(M, tx.dtype)
    op.run_raw(d, tx.data_ptr(), big.data_ptr() + pad * big.element_size(), op.workspace(d))
    torch.cuda.synchronize()
    op.ctx.device_status()
    got = big.cpu().numpy()
    assert np.isnan(got[:pad]).all() and np.isnan(got[pad + M * N:]).all()
    y = got[pad: pad + M * N].reshape(M, N)
    assert orc.max_rel_err(y, oracle_linear(x, w, out_dtype=out)) <= TOL_F16


def test_attention_leaves_the_rest_of_the_caches_alone():
    """The call appends row `position` to both caches and nothing else: rows behind it (poisoned here) stay as they
    were, rows in front of it keep their bits."""
    import torch
    from nnfusion_b200.attention import DecodeAttention
    from oracle import attention as att

    H, Hkv, cap, pos = 8, 2, 96, 40
    rng = np.random.Generator(np.random.PCG64(55))
    q, kn, vn = (rng.standard_normal((n, 128)).astype(np.float16) for n in (H, Hkv, Hkv))
    kc, vc = (rng.standard_normal((Hkv, cap, 128)).astype(np.float16) for _ in range(2))
    kc[:, pos + 1:], vc[:, pos + 1:] = np.nan, np.nan
    node = DecodeAttention(H, Hkv, 128, cap, "cuda:0")
    node.k_cache.copy_(torch.from_numpy(kc))
    node.v_cache.copy_(torch.from_numpy(vc))
    y = node(*(torch.from_numpy(a).cuda() for a in (q, kn, vn)), pos).cpu().numpy().reshape(H, 128)
    torch.cuda.synchronize()
    k_after, v_after = node.k_cache.cpu().numpy(), node.v_cache.cpu().numpy()
    assert np.isnan(k_after[:, pos + 1:]).all() and np.isnan(v_after[:, pos + 1:]).all()
    np.testing.assert_array_equal(k_after[:, :pos], kc[:, :pos])
    np.testing.assert_array_equal(v_after[:, :pos], vc[:, :pos])
    np.testing.assert_array_equal(v_after[:, pos], vn)             # the new value row, as given
    kc0, vc0 = kc.copy(), vc.copy()
    kc0[:, pos + 1:], vc0[:, pos + 1:] = 0, 0
    r, _ = att.decode_attention(q, kn, vn, kc0, vc0, pos)
    assert orc.max_rel_err(y, r) <= TOL_F16
