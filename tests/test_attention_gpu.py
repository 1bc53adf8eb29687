"""Parity of the decode-attention kernel and of the add epilogue with the CPU oracle, through the C-ABI, on a B200."""
import ctypes

import numpy as np
import pytest

from nnfusion_b200 import synth
from oracle import attention as att
from oracle import oracle as orc
from tests.util import TOL_F16

pytestmark = pytest.mark.gpu


def _run(H, Hkv, cap, pos, seed, rotary=True, splits=0, calls=1):
    import torch
    from nnfusion_b200.attention import DecodeAttention

    rng = np.random.Generator(np.random.PCG64(seed))
    D = 128
    q = rng.standard_normal((H, D)).astype(np.float16)
    kn = rng.standard_normal((Hkv, D)).astype(np.float16)
    vn = rng.standard_normal((Hkv, D)).astype(np.float16)
    kc = rng.standard_normal((Hkv, cap, D)).astype(np.float16)
    vc = rng.standard_normal((Hkv, cap, D)).astype(np.float16)
    kc[:, pos:] = 0          # rows from `pos` on are not part of the sequence yet
    vc[:, pos:] = 0
    op = DecodeAttention(H, Hkv, D, cap, "cuda:0", rotary=rotary, splits=splits)
    op.k_cache.copy_(torch.from_numpy(kc))
    op.v_cache.copy_(torch.from_numpy(vc))
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, kn, vn))
    outs = []
    for _ in range(calls):
        y = op(tq, tk, tv, pos)
        torch.cuda.synchronize()
        outs.append(y.cpu().numpy().reshape(H, D))
    op.ctx.device_status()
    kc_r, vc_r = kc.copy(), vc.copy()
    ref, k_row = att.decode_attention(q, kn, vn, kc_r, vc_r, pos, rotary=rotary)
    return outs, ref, (op.k_cache.cpu().numpy(), op.v_cache.cpu().numpy()), (kc_r, vc_r)


def _check(y, r, tol=TOL_F16):
    err = orc.max_rel_err(y, r)
    assert err <= tol, f"max rel err {err:.3e} > {tol}"


def test_config4_attention_full_size():
    # 32 heads x 2048 cached rows x 128, the new token at position 2048 (the 7B-layer decode configuration)
    outs, ref, caches, caches_ref = _run(32, 32, 2049, 2048, seed=40)
    _check(outs[0], ref)
    # the appended rows: the key through the rotary embedding rounds like the oracle's up to one fp16 ulp
    np.testing.assert_array_equal(caches[1], caches_ref[1])
    np.testing.assert_allclose(caches[0].astype(np.float32), caches_ref[0].astype(np.float32), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("pos", [0, 1, 15, 16, 31, 32, 33, 100, 777])
def test_ragged_lengths(pos):
    outs, ref, _, _ = _run(4, 4, 1024, pos, seed=41 + pos)
    _check(outs[0], ref)


@pytest.mark.parametrize("H,Hkv", [(8, 8), (8, 2), (64, 8), (3, 1), (12, 2), (10, 5), (16, 1)])
def test_grouped_queries(H, Hkv):
    """Groups of 1, 2, 3, 4, 6, 8 and 16 query heads per key/value head."""
    outs, ref, caches, caches_ref = _run(H, Hkv, 600, 555, seed=50 + H)
    _check(outs[0], ref)
    np.testing.assert_array_equal(caches[1], caches_ref[1])


def test_grouped_queries_long_cache_repeats():
    # 64 query heads on 8 key/value heads over 4097 rows (a 70B-shaped decode step), three calls: same bits
    outs, ref, _, _ = _run(64, 8, 4100, 4096, seed=59, calls=3)
    _check(outs[0], ref)
    np.testing.assert_array_equal(outs[0], outs[1])
    np.testing.assert_array_equal(outs[0], outs[2])


def test_without_rotary_and_last_row_of_the_cache():
    outs, ref, caches, caches_ref = _run(8, 8, 300, 299, seed=60, rotary=False)
    _check(outs[0], ref)
    np.testing.assert_array_equal(caches[0], caches_ref[0])   # no rotation: the key row is copied bit for bit


@pytest.mark.parametrize("splits", [1, 2, 5, 64])
def test_forced_splits_agree_and_repeat(splits):
    outs, ref, _, _ = _run(8, 4, 2048, 1500, seed=70, splits=splits, calls=3)
    _check(outs[0], ref)
    # same call, same bits (fixed summation order) -- and the workspace counters were left ready for reuse
    np.testing.assert_array_equal(outs[0], outs[1])
    np.testing.assert_array_equal(outs[0], outs[2])


def test_softmax_uniform_when_keys_are_equal():
    # the reference's softmax vector (ones -> uniform weights): equal keys make the output the mean of the values
    import torch
    from nnfusion_b200.attention import DecodeAttention

    H, D, pos = 4, 128, 199
    rng = np.random.Generator(np.random.PCG64(80))
    op = DecodeAttention(H, H, D, 256, "cuda:0", rotary=False)
    v = rng.standard_normal((H, pos + 1, D)).astype(np.float16)
    op.k_cache[:, :pos] = 1.0
    op.v_cache[:, :pos] = torch.from_numpy(v[:, :pos]).cuda()
    q = torch.from_numpy(rng.standard_normal((H, D)).astype(np.float16)).cuda()
    k_new = torch.ones((H, D), dtype=torch.float16, device="cuda")
    y = op(q, k_new, torch.from_numpy(v[:, pos]).cuda(), pos).cpu().numpy().reshape(H, D)
    np.testing.assert_allclose(y.astype(np.float32), v.astype(np.float32).mean(axis=1), rtol=0, atol=2e-3)


def test_invalid_arguments():
    from nnfusion_b200 import _lib as L
    from nnfusion_b200.attention import DecodeAttention
    from nnfusion_b200.linear import NNFB200Error
    import torch

    op = DecodeAttention(8, 8, 128, 64, "cuda:0")
    q = torch.zeros(8 * 128, dtype=torch.float16, device="cuda")
    with pytest.raises(NNFB200Error):
        op(q, q, q, 64)                       # position == capacity
    bad = DecodeAttention(8, 3, 128, 64, "cuda:0")
    with pytest.raises(NNFB200Error):
        bad(q, q[:3 * 128], q[:3 * 128], 3)   # heads not a multiple of kv_heads
    d = op.desc(5)
    d.head_dim = 64
    lib = op.ctx.lib
    rc = lib.nnf_b200_decode_attention(op.ctx.handle, None, ctypes.byref(d), q.data_ptr(), q.data_ptr(),
                                       q.data_ptr(), op.k_cache.data_ptr(), op.v_cache.data_ptr(), q.data_ptr(),
                                       None, 0)
    assert rc == L.ENOTSUP
    d = op.desc(40)
    rc = lib.nnf_b200_decode_attention(op.ctx.handle, None, ctypes.byref(d), None, q.data_ptr(), q.data_ptr(),
                                       op.k_cache.data_ptr(), op.v_cache.data_ptr(), q.data_ptr(), None, 0)
    assert rc == L.EINVAL


@pytest.mark.parametrize("M,kernel", [(1, 1), (5, 1), (16, 1), (160, 2)])
def test_add_epilogue(M, kernel):
    # MatMulAdd with a full-size addend: y = x.W^T + c, also in place (c is y)
    import torch
    from nnfusion_b200.linear import DequantDot, DeviceWeight
    from tests.util import oracle_linear

    rng = np.random.Generator(np.random.PCG64(90 + M))
    N, K = 272, 1024
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    c = rng.standard_normal((M, N)).astype(np.float16)
    ref = (oracle_linear(x, w, out_dtype=np.float32).astype(np.float32) + c.astype(np.float32)).astype(np.float16)
    op = DequantDot(DeviceWeight.from_host(w, "cuda:0"), add=True, kernel=kernel)
    tx, tc = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    y = op(tx, addend=tc)
    torch.cuda.synchronize()
    _check(y.cpu().numpy(), ref)
    y2 = op(tx, out=tc, addend=tc)           # in place
    torch.cuda.synchronize()
    np.testing.assert_array_equal(y2.cpu().numpy(), y.cpu().numpy())
    op.ctx.device_status()
