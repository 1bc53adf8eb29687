"""The per-rank linears of the 70B-shaped MLP at 4 and 8 ranks, each run alone on one GPU against the oracle: the
column shard of gate/up with the fused SiLU*mul epilogue, and the row (K) shard of down, whose K of 7168 or 3584 is
not a multiple of the kernel's 16 K slices of 256 weights."""
import numpy as np
import pytest

from nnfusion_b200 import synth
from nnfusion_b200.tp import mlp_shapes
from oracle import oracle as orc
from tests.util import TOL_F16, gpu_linear, oracle_linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("M", [1, 16])
def test_mlp70b_rank_shards(world, M):
    (n_gu, k_gu), (n_d, k_d) = mlp_shapes(8192, 28672, world)
    rng = np.random.Generator(np.random.PCG64(700 + world))
    x = synth.make_x(rng, M, k_gu, np.float16)
    gate = synth.make_weights(rng, n_gu, k_gu, 4, 128)
    up = synth.make_weights(rng, n_gu, k_gu, 4, 128)
    h = gpu_linear(x, gate, up)
    r = oracle_linear(x, gate, up)
    assert h.shape == (M, n_gu) and h.dtype == np.float16
    assert orc.max_rel_err(h, r) <= TOL_F16
    down = synth.make_weights(rng, n_d, k_d, 4, 128)
    y = gpu_linear(h, down)
    ry = oracle_linear(h, down)
    assert y.shape == (M, n_d)
    assert orc.max_rel_err(y, ry) <= TOL_F16
    # the partial sum a rank hands to the exchange is fp32 in the fused entry point: same shapes, fp32 output
    y32 = gpu_linear(h, down, out_dtype=np.float32)
    assert orc.max_rel_err(y32, oracle_linear(h, down, out_dtype=np.float32)) <= TOL_F16
