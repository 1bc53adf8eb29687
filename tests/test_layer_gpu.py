"""The 7B-shaped decoder layer at decode time (configuration 4): five fused launches against the oracle's graph."""
import numpy as np
import pytest

from nnfusion_b200 import synth
from oracle import attention as att
from oracle import oracle as orc
from tests.util import oracle_linear

pytestmark = pytest.mark.gpu


def _oracle_layer(x, W, g1, g2, kc, vc, pos, heads, kv_heads, eps=1e-6):
    """Node by node as the reference graph would run it, every node's output rounded to fp16."""
    q = oracle_linear(x, W["q"], gain=g1, eps=eps)
    k = oracle_linear(x, W["k"], gain=g1, eps=eps)
    v = oracle_linear(x, W["v"], gain=g1, eps=eps)
    D = q.shape[1] // heads
    a, _ = att.decode_attention(q.reshape(heads, D), k.reshape(kv_heads, D), v.reshape(kv_heads, D), kc, vc, pos)
    a = a.reshape(1, -1)
    x1 = (oracle_linear(a, W["o"], out_dtype=np.float32) + x.astype(np.float32)).astype(np.float16)
    h = oracle_linear(x1, W["gate"], W["up"], gain=g2, eps=eps)
    return (oracle_linear(h, W["down"], out_dtype=np.float32) + x1.astype(np.float32)).astype(np.float16)


@pytest.mark.parametrize("hidden,inter,heads,kv_heads,cap,pos", [
    (512, 1408, 4, 4, 64, 37),          # small: every path, ragged sizes
    (4096, 11008, 32, 32, 2049, 2048),  # configuration 4 at full size
])
def test_decoder_layer_against_oracle(hidden, inter, heads, kv_heads, cap, pos):
    import torch
    from nnfusion_b200.decoder_layer import DecoderLayer
    from nnfusion_b200.linear import DeviceWeight

    rng = np.random.Generator(np.random.PCG64(400 + hidden))
    D = hidden // heads
    x = synth.make_x(rng, 1, hidden, np.float16)
    shapes = {"q": (hidden, hidden), "k": (kv_heads * D, hidden), "v": (kv_heads * D, hidden), "o": (hidden, hidden),
              "gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}
    W = {n: synth.make_weights(rng, s[0], s[1], 4, 128) for n, s in shapes.items()}
    g1 = rng.uniform(0.9, 1.1, hidden).astype(np.float32)
    g2 = rng.uniform(0.9, 1.1, hidden).astype(np.float32)
    kc = rng.standard_normal((kv_heads, cap, D)).astype(np.float16)
    vc = rng.standard_normal((kv_heads, cap, D)).astype(np.float16)

    dev = "cuda:0"
    dw = {n: DeviceWeight.from_host(w, dev) for n, w in W.items()}
    layer = DecoderLayer(dw["q"], dw["k"], dw["v"], dw["o"], dw["gate"], dw["up"], dw["down"],
                         torch.from_numpy(g1).to(dev), torch.from_numpy(g2).to(dev),
                         heads=heads, kv_heads=kv_heads, capacity=cap)
    layer.attn.k_cache.copy_(torch.from_numpy(kc))
    layer.attn.v_cache.copy_(torch.from_numpy(vc))
    y = layer(torch.from_numpy(x).to(dev), pos)
    torch.cuda.synchronize()
    layer.qkv.ctx.device_status()
    ref = _oracle_layer(x, W, g1, g2, kc.copy(), vc.copy(), pos, heads, kv_heads)
    err = orc.max_rel_err(y.cpu().numpy(), ref)
    # five fp16 node boundaries: each within the fp16 gate, the layer within twice that
    assert err <= 1e-2, f"max rel err {err:.3e}"
