"""Host logic of the tensor-parallel MLP, on CPU: the sharding helpers and the all-reduce over world_size-2 gloo
ranks reproduce the unsharded oracle result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nnfusion_b200 import synth
from nnfusion_b200.tp import mlp_shapes, shard_k_of_w, shard_rows_of_w
from oracle import oracle as orc


def _mlp_inputs(seed=0, M=3, hidden=256, inter=512):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = synth.make_x(rng, M, hidden, np.float16)
    gate = synth.make_weights(rng, inter, hidden, 4, 128)
    up = synth.make_weights(rng, inter, hidden, 4, 128)
    down = synth.make_weights(rng, hidden, inter, 4, 128)
    return x, gate, up, down


def _oracle_mlp(x, gate, up, down):
    h = orc.linear(x, gate.q, gate.scale, gate.zp, 128, q2=up.q, scale2=up.scale, zp2=up.zp)   # fp16
    return orc.linear(h, down.q, down.scale, down.zp, 128, out_dtype=np.float32)


def test_shard_helpers_partition_the_weights():
    _, gate, _, down = _mlp_inputs()
    parts = [shard_rows_of_w(gate, r, 4) for r in range(4)]
    np.testing.assert_array_equal(np.concatenate([p.q for p in parts]), gate.q)
    np.testing.assert_array_equal(np.concatenate([p.scale for p in parts]), gate.scale)
    kparts = [shard_k_of_w(down, r, 2) for r in range(2)]
    np.testing.assert_array_equal(np.concatenate([p.q for p in kparts], axis=1), down.q)
    np.testing.assert_array_equal(np.concatenate([p.zp for p in kparts], axis=1), down.zp)
    assert mlp_shapes(8192, 28672, 8) == ((3584, 8192), (8192, 3584))
    with pytest.raises(ValueError):
        shard_k_of_w(down, 0, 3)
    with pytest.raises(ValueError):
        mlp_shapes(8192, 28672, 3)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, gate, up, down = _mlp_inputs()
        g, u, d = shard_rows_of_w(gate, rank, world), shard_rows_of_w(up, rank, world), shard_k_of_w(down, rank, world)
        h_local = orc.linear(x, g.q, g.scale, g.zp, 128, q2=u.q, scale2=u.scale, zp2=u.zp)        # [M, inter/world] fp16
        y_part = orc.linear(h_local, d.q, d.scale, d.zp, 128, out_dtype=np.float32)               # partial over K shard
        t = torch.from_numpy(y_part.copy())
        dist.all_reduce(t)                                                                         # the shard boundary
        if rank == 0:
            np.save(out_path, t.numpy())
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_mlp_matches_unsharded_oracle(tmp_path):
    out = str(tmp_path / "y.npy")
    mp.spawn(_rank_main, args=(2, _free_port(), out), nprocs=2, join=True)
    y = np.load(out)
    x, gate, up, down = _mlp_inputs()
    r = _oracle_mlp(x, gate, up, down)
    assert orc.max_rel_err(y, r) < 1e-5      # same fp32 partial products, summed in a different order
