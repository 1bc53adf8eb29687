"""CPU tests of the attention oracle: the reference's own vectors, its compiled MLAS, and self-consistency."""
import numpy as np
import pytest

from oracle import attention as att
from oracle import oracle as orc


def test_softmax_reference_vector():
    # test/nnfusion/frontend/torchscript_import.cpp:160-190: softmax over the last axis of ones(2,3,5) is 0.2
    y = att.softmax(np.ones((2, 3, 5), np.float32), axis=-1)
    assert y.shape == (2, 3, 5)
    np.testing.assert_allclose(y, 0.2, rtol=0, atol=1e-7)


def test_softmax_steps_follow_the_reference_kernel():
    # cpu_reference_softmax: max, exp(x - max), sum, divide -- rows sum to one, shift-invariant, no overflow
    rng = np.random.default_rng(0)
    x = rng.normal(size=(4, 7, 33)).astype(np.float32) * 30
    y = att.softmax(x)
    np.testing.assert_allclose(y.sum(-1), 1.0, rtol=0, atol=2e-6)
    np.testing.assert_allclose(att.softmax(x + 64.0), y, rtol=0, atol=1e-4)
    assert np.isfinite(y).all()


@pytest.mark.parametrize("adj_x,adj_y", [(False, False), (False, True), (True, False), (True, True)])
def test_batch_matmul_against_compiled_mlas(adj_x, adj_y):
    if not orc.have_ref():
        pytest.skip("reference MLAS not built")
    rng = np.random.default_rng(1)
    m, k, n = 3, 40, 5
    a = rng.normal(size=(2, 3) + ((k, m) if adj_x else (m, k))).astype(np.float32)
    b = rng.normal(size=(2, 3) + ((n, k) if adj_y else (k, n))).astype(np.float32)
    y = att.batch_matmul(a, b, adj_x, adj_y)
    r = att.ref_batch_matmul(a, b, adj_x, adj_y)
    assert y.shape == r.shape == (2, 3, m, n)     # shape rule of BatchMatMul.cpp:32-47
    np.testing.assert_allclose(y, r, rtol=1e-5, atol=1e-5)


def test_batch_matmul_rejects_mismatched_batches():
    with pytest.raises(ValueError):
        att.batch_matmul(np.zeros((2, 3, 4)), np.zeros((3, 4, 5)))


def test_rotate_half_is_a_rotation():
    rng = np.random.default_rng(2)
    x = rng.normal(size=(5, 128)).astype(np.float32)
    cos, sin = att.rotary_tables(2048, 128)
    y = att.rotate_half(x, cos, sin)
    np.testing.assert_allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)
    c0, s0 = att.rotary_tables(0, 128)
    np.testing.assert_array_equal(att.rotate_half(x, c0, s0), x)   # position 0: identity
    # relative-position property: <rot_p(a), rot_q(b)> depends on p - q only
    a, b = x[0], x[1]
    d1 = att.rotate_half(a, *att.rotary_tables(17, 128)) @ att.rotate_half(b, *att.rotary_tables(5, 128))
    d2 = att.rotate_half(a, *att.rotary_tables(112, 128)) @ att.rotate_half(b, *att.rotary_tables(100, 128))
    assert abs(d1 - d2) < 1e-3


def test_decode_attention_small_against_direct_formula():
    rng = np.random.default_rng(3)
    H, Hkv, D, cap, pos = 4, 2, 128, 16, 9
    q = rng.normal(size=(H, D)).astype(np.float16)
    kn = rng.normal(size=(Hkv, D)).astype(np.float16)
    vn = rng.normal(size=(Hkv, D)).astype(np.float16)
    kc = rng.normal(size=(Hkv, cap, D)).astype(np.float16)
    vc = rng.normal(size=(Hkv, cap, D)).astype(np.float16)
    kc2, vc2 = kc.copy(), vc.copy()
    out, k_row = att.decode_attention(q, kn, vn, kc2, vc2, pos)
    # the caches received the new row, nothing else changed
    np.testing.assert_array_equal(kc2[:, pos], k_row)
    np.testing.assert_array_equal(vc2[:, pos], vn)
    np.testing.assert_array_equal(kc2[:, :pos], kc[:, :pos])
    # direct float64 formula per head
    cos, sin = att.rotary_tables(pos, D)
    for h in range(H):
        g = h // (H // Hkv)
        qr = att.rotate_half(q[h].astype(np.float32), cos, sin).astype(np.float64)
        K = kc2[g, :pos + 1].astype(np.float64)
        V = vc2[g, :pos + 1].astype(np.float64)
        s = K @ qr / np.sqrt(D)
        p = np.exp(s - s.max())
        p /= p.sum()
        np.testing.assert_allclose(out[h].astype(np.float64), p @ V, rtol=0, atol=2e-3)
    if orc.have_ref():
        out_ref, _ = att.decode_attention(q, kn, vn, kc.copy(), vc.copy(), pos, use_ref=True)
        np.testing.assert_allclose(out_ref.astype(np.float32), out.astype(np.float32), rtol=0, atol=2e-3)


def test_decode_attention_first_token():
    rng = np.random.default_rng(4)
    q = rng.normal(size=(2, 128)).astype(np.float16)
    kn = rng.normal(size=(2, 128)).astype(np.float16)
    vn = rng.normal(size=(2, 128)).astype(np.float16)
    kc = np.zeros((2, 4, 128), np.float16)
    vc = np.zeros((2, 4, 128), np.float16)
    out, _ = att.decode_attention(q, kn, vn, kc, vc, 0)
    np.testing.assert_array_equal(out, vn)        # one row: the softmax weight is exactly 1
