"""Generates tests/golden/mlas_linear_small.npz: outputs of the reference's own CPU arithmetic (its vendored MLAS
SGEMM compiled in place, behind the restated Convert / Subtract / Multiply kernels: oracle/_ref) on small seeded
cases of the dequantised linear.  Run where the reference checkout is available:

    make -C oracle && python tests/golden/make_golden.py

The fixture lets the oracle be pinned on machines that have neither the reference sources nor oracle/_ref.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from nnfusion_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

CASES = {
    # name: (generator, kwargs)
    "config1_small": ("config1", dict(seed=0, M=16, N=96, K=256)),
    "u4g128_m1": ("u4g128", dict(seed=1, M=1, N=64, K=512)),
    "u4g128_m5": ("u4g128", dict(seed=2, M=5, N=48, K=384)),
}


def inputs(kind, kw):
    x, w = (synth.config1(**kw) if kind == "config1" else synth.u4g128(**kw))
    return x, w


def main():
    out = {}
    for name, (kind, kw) in CASES.items():
        x, w = inputs(kind, kw)
        graph = orc.RefLinearGraph(w.N, w.K)
        y = graph(x.astype(np.float32), w.q, w.scale.astype(np.float32), w.zp, w.group)
        out[name] = y
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "mlas_linear_small.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
