"""The one-shot all-reduce kernel on ONE GPU: all "ranks" are buffers of this GPU and the peers' flags are written by
the host beforehand, so the kernel under test never waits for another launch.  (The real thing, two processes on two
GPUs, is in test_tp_gpu.py.)"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HDR = 16  # words in front of the flag words of a flag area: call counter, ticket, padding


def _setup(world, n, seed=0):
    import torch
    from nnfusion_b200.linear import default_context

    ctx = default_context(0)
    rng = np.random.Generator(np.random.PCG64(seed))
    # two halves per rank; `parts` is what half 1 holds (odd call numbers), half 0 holds its negation
    parts = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]
    bufs = [torch.from_numpy(np.concatenate([-p, p])).cuda() for p in parts]
    fb = int(ctx.lib.nnf_b200_allreduce_flag_bytes(n))
    flags = [torch.zeros(fb // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    vp = ctypes.c_void_p
    return ctx, parts, bufs, flags, (vp * world)(*[b.data_ptr() for b in bufs]), (vp * world)(*[f.data_ptr() for f in flags])


@pytest.mark.parametrize("world,n,rank", [(2, 8192, 0), (4, 8192, 3), (8, 16 * 8192, 5), (3, 8, 1), (2, 2056, 1)])
def test_sum_in_rank_order(world, n, rank):
    import torch
    ctx, parts, bufs, flags, pb, pf = _setup(world, n, seed=world)
    epoch = 7
    flags[rank][HDR: HDR + (n // 8 + 255) // 256 * 8].fill_(epoch)   # every peer "has announced" call 7 to this rank
    out = torch.empty(n, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ctx.check(ctx.lib.nnf_b200_allreduce_oneshot(ctx.handle, s, rank, world, pb, pf, n, 2 * n, out.data_ptr(), epoch))
    torch.cuda.synchronize()
    ctx.device_status()
    acc = np.zeros(n, np.float32)
    for p in parts:                       # rank order, fp32, one rounding: bit-exact
        acc += p.astype(np.float32)
    np.testing.assert_array_equal(out.cpu().numpy(), acc.astype(np.float16))
    # the kernel announced itself to every peer, and to nobody else
    for r in range(world):
        ctas = (n // 8 + 255) // 256
        f = flags[r].cpu().numpy()[HDR: HDR + ctas * 8].reshape(-1, 8)
        if r != rank:
            assert (f[:, rank] == epoch).all() and (np.delete(f, rank, axis=1) == 0).all()


def test_device_counted_calls_alternate_halves():
    import torch
    ctx, parts, bufs, flags, pb, pf = _setup(3, 4096, seed=9)
    flags[1][HDR: HDR + 2 * 8].fill_(1000)  # the peers are "far ahead": no call of this test has to wait
    out = torch.empty(4096, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    acc = np.zeros(4096, np.float32)
    for p in parts:
        acc += p.astype(np.float32)
    for call in (1, 2, 3, 4):
        ctx.check(ctx.lib.nnf_b200_allreduce_oneshot(ctx.handle, s, 1, 3, pb, pf, 4096, 8192, out.data_ptr(), 0))
        torch.cuda.synchronize()
        ctx.device_status()
        want = acc if call & 1 else -acc    # half (call & 1)
        np.testing.assert_array_equal(out.cpu().numpy(), want.astype(np.float16))
    header = flags[1].cpu().numpy()[:2]
    assert header[0] == 4 and header[1] == 0          # four calls counted, ticket back at zero


def test_calls_of_different_sizes_share_one_flag_area():
    """One flag area, sized for the largest tensor, serves calls of 1, 2 and 1 rows of 8192 (4, 8, 4 CTAs): the call
    counter and the flag words sit where they sit whatever the size of a call, every CTA of a call takes the same
    buffer half, and CTAs that sat out a call do not fall behind."""
    import torch
    from nnfusion_b200.linear import default_context
    ctx = default_context(0)
    world, rank, row = 2, 0, 8192
    rng = np.random.Generator(np.random.PCG64(21))
    fb = int(ctx.lib.nnf_b200_allreduce_flag_bytes(2 * row))
    flags = [torch.zeros(fb // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    flags[rank][HDR:].fill_(1000)                     # the peer is "far ahead" on every flag word
    half = 2 * row * 2                                 # bytes of one buffer half (room for two rows)
    bufs = [torch.zeros(2 * 2 * row, dtype=torch.float16, device="cuda") for _ in range(world)]
    vp = ctypes.c_void_p
    pb = (vp * world)(*[b.data_ptr() for b in bufs])
    pf = (vp * world)(*[f.data_ptr() for f in flags])
    s = torch.cuda.current_stream().cuda_stream
    for call, rows in enumerate((1, 2, 1, 2, 2, 1), start=1):
        n = rows * row
        parts = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]
        for b, part in zip(bufs, parts):               # this call's addends go into half (call & 1); the other half
            b.fill_(float("nan"))                      # is poison: a CTA that took the wrong half would show it
            off = (call & 1) * 2 * row
            b[off: off + n].copy_(torch.from_numpy(part))
        out = torch.full((2 * row,), -7.0, dtype=torch.float16, device="cuda")
        ctx.check(ctx.lib.nnf_b200_allreduce_oneshot(ctx.handle, s, rank, world, pb, pf, n, half, out.data_ptr(), 0))
        torch.cuda.synchronize()
        ctx.device_status()
        want = (parts[0].astype(np.float32) + parts[1].astype(np.float32)).astype(np.float16)
        got = out.cpu().numpy()
        np.testing.assert_array_equal(got[:n], want)
        assert (got[n:] == -7.0).all()                 # nothing written past the tensor of this call
        assert int(flags[rank][0]) == call and int(flags[rank][1]) == 0
        ctas = (n // 8 + 255) // 256
        f = flags[1 - rank].cpu().numpy()[HDR:].reshape(-1, 8)
        assert (f[:ctas, rank] == call).all()          # announced to the peer with the call number


def test_later_epoch_counts_as_arrived_and_wraps():
    import torch
    ctx, parts, bufs, flags, pb, pf = _setup(2, 4096)
    out = torch.empty(4096, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for flag, epoch in ((12, 11), (3, 0xFFFFFFFE)):   # a peer one call ahead; a peer ahead across the wrap
        flags[0].fill_(flag if flag < 2**31 else flag - 2**32)
        ctx.check(ctx.lib.nnf_b200_allreduce_oneshot(ctx.handle, s, 0, 2, pb, pf, 4096, 8192, out.data_ptr(), epoch))
        torch.cuda.synchronize()
        ctx.device_status()


def test_wait_runs_out_and_context_stays_usable():
    # a flag that nobody sets: the bounded wait gives up, the status word says so, nothing is written
    import torch
    from nnfusion_b200 import _lib as L
    from nnfusion_b200.linear import NNFB200Error
    ctx, parts, bufs, flags, pb, pf = _setup(2, 4096)
    out = torch.full((4096,), 5.0, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ctx.check(ctx.lib.nnf_b200_allreduce_oneshot(ctx.handle, s, 0, 2, pb, pf, 4096, 8192, out.data_ptr(), 1))
    torch.cuda.synchronize()
    with pytest.raises(NNFB200Error) as e:
        ctx.device_status()
    assert e.value.status == L.ETIMEDOUT
    assert (out == 5.0).all()
    ctx.device_status()                   # cleared; the context still works
    flags[0].fill_(2)
    ctx.check(ctx.lib.nnf_b200_allreduce_oneshot(ctx.handle, s, 0, 2, pb, pf, 4096, 8192, out.data_ptr(), 2))
    torch.cuda.synchronize()
    ctx.device_status()


def test_invalid_arguments():
    from nnfusion_b200 import _lib as L
    ctx, parts, bufs, flags, pb, pf = _setup(2, 4096)
    lib, h = ctx.lib, ctx.handle
    o = bufs[0].data_ptr()
    assert lib.nnf_b200_allreduce_oneshot(h, None, 0, 9, pb, pf, 4096, 8192, o, 1) == L.EINVAL
    assert lib.nnf_b200_allreduce_oneshot(h, None, 2, 2, pb, pf, 4096, 8192, o, 1) == L.EINVAL
    assert lib.nnf_b200_allreduce_oneshot(h, None, 0, 2, pb, pf, 4096, 100, o, 1) == L.EINVAL
    assert lib.nnf_b200_allreduce_oneshot(h, None, 0, 2, pb, pf, 4100, 16384, o, 1) == L.ENOTSUP
    assert lib.nnf_b200_allreduce_oneshot(h, None, 0, 2, pb, pf, 4096, 8192, o + 2, 1) == L.EALIGN


@pytest.mark.parametrize("M,N,K,world,rank", [(1, 272, 1024, 2, 0), (16, 96, 512, 3, 1), (3, 512, 4608, 4, 2)])
def test_linear_with_fused_sum_over_ranks(M, N, K, world, rank):
    """nnf_b200_linear_allreduce on one GPU: this rank's buffer holds known partial sums in the peers' slots (a rank
    writes its sums into every rank's buffer) and their flags were set by the host, so nothing waits; K = 4608
    exercises split-K (the last-arriving split does the exchange)."""
    import torch
    from nnfusion_b200 import _lib as L
    from nnfusion_b200 import synth
    from nnfusion_b200.linear import DequantDot, DeviceWeight
    from tests.util import oracle_linear

    rng = np.random.Generator(np.random.PCG64(1000 + M))
    x = synth.make_x(rng, M, K, np.float16)
    w = synth.make_weights(rng, N, K, 4, 128)
    node = DequantDot(DeviceWeight.from_host(w, "cuda:0"))
    ctx = node.ctx
    half = (world * M * N * 4 + 255) // 256 * 256       # one M x N block per sender
    d = node.desc(M, torch.float16)
    fb = int(ctx.lib.nnf_b200_linear_allreduce_flag_bytes(ctypes.byref(d)))
    others = [rng.standard_normal((M, N)).astype(np.float32) for _ in range(world)]
    bufs, flags = [], []
    for r in range(world):
        b = torch.zeros(2 * half // 4, dtype=torch.float32, device="cuda")
        bufs.append(b)
        f = torch.zeros(fb // 4, dtype=torch.int32, device="cuda")
        flags.append(f)
    for r in range(world):
        if r != rank:                                    # what peer r would have written into this rank's buffer
            bufs[rank][r * M * N: (r + 1) * M * N] = torch.from_numpy(-others[r].reshape(-1)).cuda()   # half 0: even calls
            bufs[rank][half // 4 + r * M * N: half // 4 + (r + 1) * M * N] = torch.from_numpy(others[r].reshape(-1)).cuda()
    tiles = (N + 15) // 16
    flags[rank][: tiles * 8].fill_(1000)      # the peers are far ahead: no wait in this test
    vp = ctypes.c_void_p
    pb = (vp * world)(*[b.data_ptr() for b in bufs])
    pf = (vp * world)(*[f.data_ptr() for f in flags])
    peers = L.Peers(rank, world, pb, pf, half, 0)
    tx = torch.from_numpy(x).cuda()
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ws = node.workspace(d)
    own = oracle_linear(x, w, out_dtype=np.float32).astype(np.float32)
    s = torch.cuda.current_stream().cuda_stream
    for call in (1, 2, 3):
        ctx.check(ctx.lib.nnf_b200_linear_allreduce(
            ctx.handle, s, ctypes.byref(d), tx.data_ptr(), ctypes.byref(node._abi_w), None, y.data_ptr(),
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, ctypes.byref(peers)))
        torch.cuda.synchronize()
        ctx.device_status()
        sign = 1.0 if call & 1 else -1.0
        ref = own + sign * sum(others[r] for r in range(world) if r != rank)
        err = np.abs(y.cpu().numpy().astype(np.float32) - ref).max() / np.abs(ref).max()
        assert err <= 5e-3, (call, err)
    # the device counted three calls for every tile, and told every peer so
    assert (flags[rank].cpu().numpy()[tiles * 8: tiles * 9] == 3).all()
    for r in range(world):
        if r != rank:
            assert (flags[r].cpu().numpy()[: tiles * 8].reshape(tiles, 8)[:, rank] == 3).all()
            # ... and left its own sums in the peer's buffer, slot `rank`, half 1 (call 3) and half 0 (call 2)
            for h in (0, 1):
                got = bufs[r].cpu().numpy()[h * (half // 4) + rank * M * N: h * (half // 4) + (rank + 1) * M * N]
                assert np.abs(got.reshape(M, N) - own).max() / np.abs(own).max() <= 2e-3


def test_fused_sum_rejects_what_it_does_not_serve():
    import torch
    from nnfusion_b200 import _lib as L
    from nnfusion_b200 import synth
    from nnfusion_b200.linear import DequantDot, DeviceWeight

    x, w = synth.u4g128(7, 32, 64, 256)
    node = DequantDot(DeviceWeight.from_host(w, "cuda:0"))
    ctx = node.ctx
    d = node.desc(32, torch.float16)      # 32 rows: not the small-M kernel
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    vp = ctypes.c_void_p
    pb, pf = (vp * 2)(buf.data_ptr(), buf.data_ptr()), (vp * 2)(buf.data_ptr(), buf.data_ptr())
    peers = L.Peers(0, 2, pb, pf, 32 * 64 * 4, 1)
    rc = ctx.lib.nnf_b200_linear_allreduce(ctx.handle, None, ctypes.byref(d), buf.data_ptr(),
                                           ctypes.byref(node._abi_w), None, buf.data_ptr(), None, 0, ctypes.byref(peers))
    assert rc == L.ENOTSUP
    d = node.desc(4, torch.float16)
    peers = L.Peers(2, 2, pb, pf, 4 * 64 * 4, 1)
    rc = ctx.lib.nnf_b200_linear_allreduce(ctx.handle, None, ctypes.byref(d), buf.data_ptr(),
                                           ctypes.byref(node._abi_w), None, buf.data_ptr(), None, 0, ctypes.byref(peers))
    assert rc == L.EINVAL
