"""bench.py's CPU legs: the reference arm prints the contract's JSON line, and the GPU arm refuses to run without a
device instead of falling back to anything on the CPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*argv, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *argv], cwd=ROOT, env=e,
                          capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("gpus, workload, scaling", [(1, "decode_gemv", "weak"), (2, "mlp70b_decode", "strong")])
def test_reference_arm_line(gpus, workload, scaling):
    p = run_bench("--impl", "reference", "--gpus", str(gpus), "--steps", "2", "--warmup", "1")
    assert p.returncode == 0, p.stderr
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == gpus and line["steps"] == 2 and line["warmup"] == 1
    assert line["metric"] == "int4_g128_decode_gemv_hbm_gbs" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["scaling"] == scaling and line["vs_baseline"] is None
    assert line["config"]["workload"].startswith(workload)
    assert line["value"] > 0 and line["ms_per_step"] > 0
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_do_nothing():
    p = run_bench("--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1",
                  env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert p.returncode == 0 and p.stdout.strip() == ""


def test_reference_arm_prefill_is_tflops():
    p = run_bench("--impl", "reference", "--workload", "prefill_gemm", "--steps", "1", "--warmup", "1")
    assert p.returncode == 0, p.stderr
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["metric"] == "int4_g128_prefill_gemm_tflops" and line["unit"] == "TFLOP/s" and line["value"] > 0


def test_gpu_arm_has_no_cpu_path():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = run_bench("--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert "no CUDA device" in json.loads(p.stdout.strip().splitlines()[-1])["error"]
