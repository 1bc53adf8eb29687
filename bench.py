#!/usr/bin/env python
"""Benchmark of the dequantize-fused low-bit linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  Workloads (``--workload``; ``auto`` picks by ``--gpus``):

  decode_gemv     (1 GPU, default)  uint4 group-128 decode GEMV: X fp16 [1,4096], W [11008,4096]; a step is one call of
                  the fused linear on the next of 12 weight copies (282 MB in rotation, larger than L2), so every step
                  reads its weights from HBM.  value = algorithmic bytes / time in GB/s.
  mlp70b_decode   (N GPUs, default for N > 1)  LLaMA-70B-shaped SwiGLU MLP at M = 1, uint4 group-128: gate/up split
                  by column, down by row, the fp16 [1,8192] output summed by the one-shot all-reduce kernel over peer
                  memory; a step is the whole MLP (366 MB of weights, larger than L2).  value = algorithmic bytes of
                  the whole job / time, GB/s.
  prefill_gemm    (1 GPU)  uint4 group-128 GEMM, X fp16 [4096,4096], W [11008,4096]; value in TFLOP/s.
  layer7b_decode  (1 GPU)  one LLaMA-7B-shaped decoder layer at decode time, 2048 cached rows: five launches per step.

``--impl reference`` times the reference's own CPU path for the same workload (vendored MLAS SGEMM behind the
Convert / Subtract / Multiply kernels its CPU code generation emits, all host threads) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126e6
# DRAM bytes (read + written) of one launch of the small-M kernel on the decode_gemv workload, from one ncu capture
# of that launch (dram__bytes_read.sum + dram__bytes_write.sum; the output stays in L2).
NCU_TRAFFIC_DECODE_GEMV = 23_499_008


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                r = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                    "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if r.returncode == 0 and r.stdout.strip():
                    self.rows.append([c.strip() for c in r.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        reasons = []
        for name, col in (("hw_slowdown", 3), ("hw_thermal_slowdown", 4), ("sw_thermal_slowdown", 5), ("sw_power_cap", 6)):
            if any(r[col] == "Active" for r in self.rows if len(r) > col):
                reasons.append(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": float(self.rows[0][1]),
                "reasons": reasons, "samples": len(self.rows)}


def rand_device_weight(torch, N, K, bits=4, group=128, scale_dtype=None, device="cuda", seed=None):
    """Random quantised weights generated on the device (content does not matter for timing; with `seed` every rank
    gets the same tensors)."""
    from nnfusion_b200.linear import DeviceWeight
    scale_dtype = scale_dtype or torch.float16
    G = K // group
    gen = None
    if seed is not None:
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
    wq = torch.randint(0, 256, (N, K // 2 if bits == 4 else K), dtype=torch.uint8, device=device, generator=gen)
    sc = (torch.rand((N, G), device=device, generator=gen) * 0.018 + 0.002).to(scale_dtype)
    zp = torch.randint(0, 256, (N, (G + 1) // 2 if bits == 4 else G), dtype=torch.uint8, device=device, generator=gen)
    return DeviceWeight(N, K, bits, group, wq, sc, zp)


def linear_bytes(M, N, K, bits=4, group=128, act_bytes=2, scale_bytes=2):
    """Algorithmic bytes of one linear: packed weights + scales + zero-points + x + y, each once."""
    G = K // group
    return N * K * bits // 8 + N * G * scale_bytes + N * ((G + 1) // 2 if bits == 4 else G) + M * K * act_bytes + M * N * act_bytes


class ExchangeUnhealthy(RuntimeError):
    """A bounded wait of a peer-memory exchange gave up on some rank during the warm-up (raised on every rank)."""


def ranks_healthy(torch, dist, ctx):
    """True when no rank's context has recorded a device-side wait that gave up (synchronises; every rank gets the
    same answer, so all of them take the same branch afterwards)."""
    ok = 1
    try:
        ctx.device_status()
    except Exception as e:  # the status call raises with the kernel's record of where it gave up
        sys.stderr.write(f"[bench] device status: {e}\n")
        ok = 0
    t = torch.tensor([ok], device="cuda", dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


REPEATS = 31  # timed passes over the K captured steps; the median pass is reported


def timed_graph_steps(torch, step_fns, steps, warmup, dist=None, health=None, repeats=REPEATS):
    """Runs `steps` steps (step i calls step_fns[i % len]) replayed from CUDA graphs, `repeats` times over, each pass
    timed with CUDA events on the launching stream between barrier + synchronize on both sides (several ranks: the
    maximum over ranks of every pass).  Returns the median pass in milliseconds.
    `health` (several ranks only) is asked after the plain warm-up steps and after a first short graph replay; when
    it answers False the function raises ExchangeUnhealthy instead of replaying thousands of steps whose waits
    would each run to their limit."""
    n = len(step_fns)
    stream = torch.cuda.Stream()
    chunk = min(steps, max(n, (1200 // n) * n))  # a multiple of n unless it is all of the steps
    graphs = {}

    def graph_of(count):
        if count not in graphs:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(count):
                    step_fns[i % n]()
            graphs[count] = g
        return graphs[count]

    with torch.cuda.stream(stream):
        if dist is not None:
            torch.cuda.synchronize()
            dist.barrier()  # set-up takes a different time on every rank; the steps' exchanges have bounded waits
        for i in range((max(warmup, 3) + 1) // 2 * 2 if health is not None else max(warmup, 3)):
            step_fns[i % n]()
        torch.cuda.synchronize()
        if health is not None:
            if not health():
                raise ExchangeUnhealthy("during the plain warm-up steps")
            probe = graph_of(2)  # an even number of steps: the exchanges' two buffer halves stay in step
            dist.barrier()
            for _ in range(3):
                probe.replay()
            torch.cuda.synchronize()
            if not health():
                raise ExchangeUnhealthy("during the first graph replays")
        full, rem = divmod(steps, chunk)
        g_full = graph_of(chunk) if full else None
        g_rem = graph_of(rem) if rem else None
        # graph warm-up: brings the clocks up and pages everything in.  With several ranks every rank must replay
        # the same number of times (the steps contain exchanges between the ranks: a rank that stopped earlier would
        # leave the others waiting for it), so the count is fixed there instead of timed.
        if dist is None:
            t0 = time.time()
            while time.time() - t0 < 0.5:
                (g_full or g_rem).replay()
                torch.cuda.synchronize()
        else:
            dist.barrier()  # capture takes a different time on every rank: start the replays together
            for _ in range(max(3, 4000 // max(1, chunk))):
                (g_full or g_rem).replay()
            torch.cuda.synchronize()
        passes = []
        for _ in range(max(1, repeats)):
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(full):
                g_full.replay()
            if g_rem is not None:
                g_rem.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            passes.append(e0.elapsed_time(e1))
    if dist is not None:
        t = torch.tensor(passes, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        passes = [float(v) for v in t.tolist()]
    return statistics.median(passes)


def timed_plain_steps(torch, step_fn, steps, warmup, dist=None):
    """Same contract without graph capture (used where a step contains a collective or host copies)."""
    if dist is not None:
        torch.cuda.synchronize()
        dist.barrier()
    for i in range(max(warmup, 3)):
        step_fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


# ----------------------------------------------------------------------------------------------- CPU reference path
def cpu_reference_gemv(seconds_budget: float, rows: int, K: int = 4096, M: int = 1, steps=None, warmup: int = 1,
                       warm_seconds: float = 2.0):
    """Times the reference CPU graph (oracle/_ref: MLAS behind restated element-wise kernels; falls back to the C
    restatement) on a `rows`-row sample of the uint4 group-128 linear.  Returns (seconds per step, steps, cores, kind)."""
    import numpy as np
    from oracle import oracle as orc
    rng = np.random.Generator(np.random.PCG64(0))
    x = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16).astype(np.float32)
    q = rng.integers(0, 16, size=(rows, K), dtype=np.uint8)          # nibbles unpacked, as the graph sees them
    scale = rng.uniform(0.002, 0.02, size=(rows, K // 128)).astype(np.float16).astype(np.float32)
    zp = rng.integers(0, 16, size=(rows, K // 128), dtype=np.uint8)
    if orc.have_ref():
        graph = orc.RefLinearGraph(rows, K)
        fn = lambda: graph(x, q, scale, zp, 128)
        cores, kind = orc.ref_threads(), "reference"
    else:
        fn = lambda: orc.linear(x, q, scale, zp, 128, out_dtype=np.float32)
        cores, kind = os.cpu_count() or 1, "port"
    # warm: at least `warmup` calls and `warm_seconds` of them (thread pool up, pages touched, caches and clocks
    # settled), so that a short timed run measures the same state as a long one
    t_warm, n_warm = time.perf_counter(), 0
    while n_warm < max(1, warmup) or time.perf_counter() - t_warm < warm_seconds:
        fn()
        n_warm += 1
    times = []
    t_start = time.perf_counter()
    i = 0
    while True:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
        i += 1
        if steps is not None and i >= steps:
            break
        if steps is None and (time.perf_counter() - t_start > seconds_budget and i >= 5):
            break
    return sum(times) / len(times), len(times), cores, kind


def cpu_reference_gemm_only(rows: int, K: int = 4096, M: int = 1, calls: int = 20):
    """Seconds per call of the SGEMM alone on already dequantised fp32 weights: what the reference's CPU graph runs
    per call when its constant folding has materialised the weights.  None without the compiled reference."""
    import numpy as np
    from oracle import oracle as orc
    if not orc.have_ref():
        return None
    rng = np.random.Generator(np.random.PCG64(0))
    x = rng.standard_normal((M, K), dtype=np.float32)
    graph = orc.RefLinearGraph(rows, K)
    graph(x, rng.integers(0, 16, size=(rows, K), dtype=np.uint8),
          rng.uniform(0.002, 0.02, size=(rows, K // 128)).astype(np.float32),
          rng.integers(0, 16, size=(rows, K // 128), dtype=np.uint8), 128)   # leaves the dequantised weights behind
    graph.gemm_only(x)
    t0 = time.perf_counter()
    for _ in range(calls):
        graph.gemm_only(x)
    return (time.perf_counter() - t0) / calls


# ----------------------------------------------------------------------------------------------- workloads (ours)
def run_decode_gemv(args, torch, sampler_index):
    from nnfusion_b200.linear import DequantDot, default_context
    N, K, M = 11008, 4096, 1
    ncopies = 12
    ctx = default_context(torch.cuda.current_device())
    ops = [DequantDot(rand_device_weight(torch, N, K)) for _ in range(ncopies)]
    x = torch.randn(M, K, device="cuda").to(torch.float16)
    y = torch.empty(M, N, device="cuda", dtype=torch.float16)
    step_fns = [(lambda op=op: op(x, y)) for op in ops]
    ctx.launch_count(reset=True)
    with ClockSampler(sampler_index) as cs:
        ms = timed_graph_steps(torch, step_fns, args.steps, args.warmup)
    ctx.device_status()
    bytes_step = linear_bytes(M, N, K)
    value = bytes_step * args.steps / (ms * 1e-3) / 1e9

    # end to end through the call a user of the generated runtime makes with host buffers (kernel_entry_host): the
    # node's host entry copies pinned host x to the device, runs the fused linear and copies y back to pinned host
    # memory (one graph launch), then synchronises -- every step.
    xh = torch.randn(M, K).to(torch.float16).pin_memory()
    yh = torch.empty(M, N, dtype=torch.float16).pin_memory()
    e2e_steps = min(args.steps, 2000)
    e2e_path, runtimes = None, []
    try:
        # The reference-facing way in: a generated nnfusion_rt project for this graph (built with nvcc against the
        # library), opened like the reference's Executor opens one, its kernel_entry_host called with host buffers.
        # One instance per weight copy (separate files, so that each has its own globals and memory pool).
        runtimes = generated_runtimes(torch, ops, M, ncopies)
        import ctypes
        xp = ctypes.cast(xh.data_ptr(), ctypes.POINTER(ctypes.c_uint16))
        yp = ctypes.cast(yh.data_ptr(), ctypes.POINTER(ctypes.c_uint16))
        entries = [rt.lib.kernel_entry_host for rt in runtimes]
        for e in entries:
            e.argtypes = [ctypes.POINTER(ctypes.c_uint16)] * 2
            e(xp, yp)
        ms_e2e = timed_plain_steps(torch, lambda i: entries[i % ncopies](xp, yp), e2e_steps, args.warmup)
        e2e_path = ("generated nnfusion_rt (nnfusion_b200.codegen, nvcc, linked against libnnf_b200.so) loaded the "
                    "reference Executor's way; kernel_entry_host: pinned host x -> device (copy), nnf_b200_linear "
                    "storing y straight into the pinned host buffer over PCIe, stream sync, per step")
    except Exception as e:  # no nvcc on this box, or the build failed: the node's own host entry instead
        sys.stderr.write(f"[bench] generated runtime unavailable ({e}); end-to-end leg through DequantDot.host_entry\n")
        for op in ops:
            op.host_entry(xh, yh)          # captures each node's graph outside the timed region
        ms_e2e = timed_plain_steps(torch, lambda i: ops[i % ncopies].host_entry(xh, yh), e2e_steps, args.warmup)
        e2e_path = ("DequantDot.host_entry: pinned host x -> device, nnf_b200_linear, device y -> pinned host "
                    "(one graph launch), stream sync, per step")
    e2e_value = bytes_step * e2e_steps / (ms_e2e * 1e-3) / 1e9
    for rt in runtimes:
        rt.close()
    peaks = measured_peaks()
    out = {
        "metric": "int4_g128_decode_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
        "ms_per_step": ms / args.steps, "repeats": REPEATS, "dtype": "f16", "scaling": "weak",
        "config": {"workload": "decode_gemv: X f16 [1,4096], W u4-g128 [11008,4096], Y f16, f32 accumulate",
                   "algorithmic_bytes_per_step": bytes_step,
                   "l2": f"rotation over {ncopies} weight copies ({ncopies * bytes_step / 1e6:.0f} MB) larger than L2",
                   "launch": "CUDA graph replay of the C-ABI calls"},
        "roofline": {"bound": "hbm", "achieved": round(value, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(value / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC_DECODE_GEMV,
                     "peak_source": f"of {peaks['source']}", "kernel": "dq_gemv_direct_kernel<4,1,false,false,2,1,true>"},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                "path": e2e_path},
        "gpu_launches": args.steps, "clocks": cs.summary(),
    }
    return out, ops, x, y


def run_config1_gemv(args, torch, sampler_index):
    """Configuration 1, the reference's own CPU-runnable case: X f32 [16,4096], W u8 [4096,4096], one f32 scale and
    one u8 zero-point per output row, Y f32.  Same contract as the headline; the end-to-end leg goes through
    DequantDot.host_entry (pinned host x -> device, the call, y -> pinned host as one graph launch, then a sync)."""
    from nnfusion_b200.linear import DequantDot, default_context
    N, K, M, ncopies = 4096, 4096, 16, 12
    ctx = default_context(torch.cuda.current_device())
    ops = [DequantDot(rand_device_weight(torch, N, K, bits=8, group=K, scale_dtype=torch.float32)) for _ in range(ncopies)]
    x = torch.randn(M, K, device="cuda")
    y = torch.empty(M, N, device="cuda")
    ctx.launch_count(reset=True)
    with ClockSampler(sampler_index) as cs:
        ms = timed_graph_steps(torch, [(lambda op=op: op(x, y)) for op in ops], args.steps, args.warmup)
    ctx.device_status()
    bytes_step = linear_bytes(M, N, K, bits=8, group=K, act_bytes=4, scale_bytes=4)
    value = bytes_step * args.steps / (ms * 1e-3) / 1e9
    xh, yh = torch.randn(M, K).pin_memory(), torch.empty(M, N).pin_memory()
    for op in ops:
        op.host_entry(xh, yh)
    e2e_steps = min(args.steps, 2000)
    ms_e2e = timed_plain_steps(torch, lambda i: ops[i % ncopies].host_entry(xh, yh), e2e_steps, args.warmup)
    peaks = measured_peaks()
    return {
        "metric": "u8_perchannel_f32_m16_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
        "ms_per_step": ms / args.steps, "repeats": REPEATS, "dtype": "f32", "scaling": "weak",
        "config": {"workload": "config1_gemv: X f32 [16,4096], W u8 per-channel [4096,4096], f32 scales, Y f32, f32 accumulate",
                   "algorithmic_bytes_per_step": bytes_step,
                   "l2": f"rotation over {ncopies} weight copies ({ncopies * bytes_step / 1e6:.0f} MB) larger than L2",
                   "launch": "CUDA graph replay of the C-ABI calls"},
        "roofline": {"bound": "hbm", "achieved": round(value, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(value / peaks["hbm_gbs"], 4), "traffic": None,
                     "peak_source": f"of {peaks['source']}", "kernel": "dq_gemv_direct_kernel<8,2,true,false,2,2,false>"},
        "e2e": {"value": round(bytes_step * e2e_steps / (ms_e2e * 1e-3) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4, "ms_per_step": ms_e2e / e2e_steps,
                "steps": e2e_steps, "path": "DequantDot.host_entry: pinned host x -> device, nnf_b200_linear, device y -> "
                                            "pinned host (one graph launch), stream sync, per step"},
        "gpu_launches": args.steps, "clocks": cs.summary(),
    }


def generated_runtimes(torch, ops, M, ncopies):
    """One generated nnfusion_rt instance per weight copy of `ops` (the weights are read back from the device and
    written as the project's Constant/*.bin): generated and built once, the shared object copied per instance."""
    import shutil
    import tempfile

    import numpy as np

    from nnfusion_b200 import codegen, runtime_loader
    from nnfusion_b200.synth import QuantLinear

    base = tempfile.mkdtemp(prefix="nnf_rt_")
    out = []
    first = None
    for i in range(ncopies):
        w = ops[i].w
        # the packed tensors as they are on the device (the generator dumps them again as Constant/*.bin)
        host = QuantLinear.from_packed(w.N, w.K, w.bits, w.group, w.wq.cpu().numpy(), w.scale.cpu().numpy(),
                                       w.zp.cpu().numpy())
        d = os.path.join(base, f"rt{i}")
        codegen.generate(d, codegen.DequantDotNode("DequantDot_0", M, host))
        if first is None:
            codegen.build(d)
            first = d
        else:
            shutil.copy(os.path.join(first, "libnnfusion_naive_rt.so"), os.path.join(d, f"libnnfusion_naive_{i}_rt.so"))
        out.append(runtime_loader.RuntimeExecutor(d))
    return out


def extra_measurements(torch, budget_s=90.0):
    """Other regimes of the same path at 1 GPU, reported beside the headline (each a few hundred ms of GPU time)."""
    from nnfusion_b200.linear import DequantDot
    peaks = measured_peaks()
    also = {}
    t_begin = time.time()

    def gemv(name, M, N, K, ncopies, bits=4, group=128, xdt=torch.float16, sdt=torch.float16, dual=False, gain=False, steps=600):
        if time.time() - t_begin > budget_s:
            return
        ops = []
        for _ in range(ncopies):
            w = rand_device_weight(torch, N, K, bits, group, sdt)
            w2 = rand_device_weight(torch, N, K, bits, group, sdt) if dual else None
            g = (torch.rand(K, device="cuda") + 0.5) if gain else None
            ops.append(DequantDot(w, w2, gain=g))
        x = torch.randn(M, K, device="cuda").to(xdt)
        y = torch.empty(M, N, device="cuda", dtype=xdt)
        ms = timed_graph_steps(torch, [(lambda op=op: op(x, y)) for op in ops], steps, 3, repeats=9)
        b = linear_bytes(M, N, K, bits, group, x.element_size(), 2 if sdt == torch.float16 else 4)
        if dual:
            b += b - M * K * x.element_size() - M * N * x.element_size()
        gbs = b * steps / (ms * 1e-3) / 1e9
        also[name] = {"us": round(ms * 1e3 / steps, 2), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4)}

    def gemm(name, M, N, K, dual=False, steps=20):
        if time.time() - t_begin > budget_s:
            return
        w = rand_device_weight(torch, N, K)
        w2 = rand_device_weight(torch, N, K) if dual else None
        op = DequantDot(w, w2)
        x = torch.randn(M, K, device="cuda").to(torch.float16)
        y = torch.empty(M, N, device="cuda", dtype=torch.float16)
        ms = timed_plain_steps(torch, lambda i: op(x, y), steps, 5)
        tf = 2.0 * M * N * K * (2 if dual else 1) * steps / (ms * 1e-3) / 1e12
        also[name] = {"us": round(ms * 1e3 / steps, 1), "TFLOP/s": round(tf, 1),
                      "frac_of_bf16_burst_peak": round(tf / peaks["bf16_tflops"], 4),
                      "frac_of_bf16_sustained_peak": round(tf / peaks["bf16_tflops_sustained"], 4)}
        if M <= 256:
            # a launch this short is partly host-bound when every call goes through Python: the same calls replayed
            # from a CUDA graph, as a serving loop would issue them
            gsteps = 6 * steps
            msg = timed_graph_steps(torch, [lambda: op(x, y)], gsteps, 5, repeats=7)
            tfg = 2.0 * M * N * K * (2 if dual else 1) * gsteps / (msg * 1e-3) / 1e12
            also[name].update({"us_graph_replay": round(msg * 1e3 / gsteps, 1),
                               "frac_of_bf16_burst_peak_graph_replay": round(tfg / peaks["bf16_tflops"], 4)})
            if M <= 64:
                # this few batch rows are bound by the weight bytes, not by the tensor core: the HBM fraction as well
                gbs = linear_bytes(M, N, K) * gsteps / (msg * 1e-3) / 1e9
                also[name]["frac_of_hbm_peak_graph_replay"] = round(gbs / peaks["hbm_gbs"], 4)

    def layer7b(name, copies=2, steps=200):
        """Configuration 4: one 7B-shaped decoder layer at decode time, 2048 cached rows, the token at position
        2048.  Algorithmic bytes: packed weights + scales + zero-points of the 7 projections, both caches read
        once, activations.  Rotation over `copies` layers (weights + caches 139 MB each) defeats L2."""
        if time.time() - t_begin > budget_s:
            return
        from nnfusion_b200.decoder_layer import DecoderLayer
        H, I, heads, pos = 4096, 11008, 32, 2048
        layers = []
        for _ in range(copies):
            W = [rand_device_weight(torch, n, k) for n, k in ((H, H), (H, H), (H, H), (H, H), (I, H), (I, H), (H, I))]
            g1, g2 = (torch.rand(H, device="cuda") * 0.2 + 0.9 for _ in range(2))
            layer = DecoderLayer(*W, g1, g2, heads=heads, kv_heads=heads, capacity=pos + 1)
            layer.attn.k_cache.normal_()
            layer.attn.v_cache.normal_()
            layers.append(layer)
        x = torch.randn(1, H, device="cuda").to(torch.float16)
        y = torch.empty_like(x)
        ms = timed_graph_steps(torch, [(lambda l=l: l(x, pos, out=y)) for l in layers], steps, 3, repeats=9)
        kv = 2 * heads * pos * 128 * 2
        b = layers[0].weight_bytes + kv + 2 * (3 * H + H + H + 2 * H + I + I + H)
        gbs = b * steps / (ms * 1e-3) / 1e9
        also[name] = {"us": round(ms * 1e3 / steps, 2), "GB/s": round(gbs, 1), "launches_per_layer": layers[0].launches,
                      "algorithmic_bytes": b, "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4)}

    def attention(name, copies=6, steps=600):
        if time.time() - t_begin > budget_s:
            return
        from nnfusion_b200.attention import DecodeAttention
        heads, pos = 32, 2048
        ops = []
        for _ in range(copies):
            op = DecodeAttention(heads, heads, 128, pos + 1)
            op.k_cache.normal_()
            op.v_cache.normal_()
            ops.append(op)
        q, k, v = (torch.randn(heads * 128, device="cuda").to(torch.float16) for _ in range(3))
        out = torch.empty((1, heads * 128), dtype=torch.float16, device="cuda")
        ms = timed_graph_steps(torch, [(lambda op=op: op(q, k, v, pos, out=out)) for op in ops], steps, 3, repeats=9)
        b = 2 * heads * (pos + 1) * 128 * 2 + 4 * heads * 128 * 2
        gbs = b * steps / (ms * 1e-3) / 1e9
        also[name] = {"us": round(ms * 1e3 / steps, 2), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4)}

    def mlp70b_one_gpu(name, steps=200):
        """The N > 1 workload (whole 70B-shaped MLP at M = 1) on this one GPU, with the same byte count: the
        one-GPU point of that strong-scaling series."""
        if time.time() - t_begin > budget_s:
            return
        from nnfusion_b200.tp import ShardedMLP
        hidden, inter, M = 8192, 28672, 1
        mlps = [ShardedMLP(rand_device_weight(torch, inter, hidden), rand_device_weight(torch, inter, hidden),
                           rand_device_weight(torch, hidden, inter)) for _ in range(2)]
        x = torch.randn(M, hidden, device="cuda").to(torch.float16)
        ms = timed_graph_steps(torch, [(lambda m=m: m(x)) for m in mlps], steps, 3, repeats=9)
        full = 2 * (linear_bytes(M, inter, hidden) - M * hidden * 2 - M * inter * 2) + M * hidden * 2 + \
            2 * M * inter * 2 + linear_bytes(M, hidden, inter) - M * inter * 2
        gbs = full * steps / (ms * 1e-3) / 1e9
        also[name] = {"us": round(ms * 1e3 / steps, 2), "GB/s": round(gbs, 1), "algorithmic_bytes": full,
                      "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4),
                      "note": "same workload and value formula as the --gpus N > 1 lines (mlp70b_decode)"}

    gemv("decode_gemv_down_4096x11008", 1, 4096, 11008, 12)
    gemv("config1_u8_perchannel_f32_m16_4096x4096", 16, 4096, 4096, 12, bits=8, group=4096, xdt=torch.float32, sdt=torch.float32)
    gemv("mlp70b_gate_up_silu_m1_28672x8192", 1, 28672, 8192, 2, dual=True, steps=100)
    gemv("mlp70b_down_m1_8192x28672", 1, 8192, 28672, 3, steps=150)
    attention("decode_attention_32x2048x128")
    layer7b("layer7b_decode_pos2048")
    mlp70b_one_gpu("mlp70b_decode_whole_mlp_m1_one_gpu")
    for M in (32, 256, 1024, 4096):     # 32: the 64-row batch tile of the tensor-core kernel
        gemm(f"prefill_gemm_up_m{M}_11008x4096", M, 11008, 4096)
    gemm("prefill_gemm_down_m4096_4096x11008", 4096, 4096, 11008)
    return also


def run_prefill_gemm(args, torch, sampler_index):
    from nnfusion_b200.linear import DequantDot, default_context
    M, N, K = 4096, 11008, 4096
    ctx = default_context(torch.cuda.current_device())
    op = DequantDot(rand_device_weight(torch, N, K))
    x = torch.randn(M, K, device="cuda").to(torch.float16)
    y = torch.empty(M, N, device="cuda", dtype=torch.float16)
    with ClockSampler(sampler_index) as cs:
        ms = timed_plain_steps(torch, lambda i: op(x, y), args.steps, args.warmup)
    ctx.device_status()
    tf = 2.0 * M * N * K * args.steps / (ms * 1e-3) / 1e12
    peaks = measured_peaks()
    xh = torch.randn(M, K).to(torch.float16).pin_memory()
    yh = torch.empty(M, N, dtype=torch.float16).pin_memory()

    def e2e_step(i):
        x.copy_(xh, non_blocking=True)
        op(x, y)
        yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(args.steps, 50)
    ms_e2e = timed_plain_steps(torch, e2e_step, e2e_steps, 3)
    return {
        "metric": "int4_g128_prefill_gemm_tflops", "value": round(tf, 1), "unit": "TFLOP/s",
        "ms_per_step": ms / args.steps, "dtype": "f16", "scaling": "weak",
        "config": {"workload": "prefill_gemm: X f16 [4096,4096], W u4-g128 [11008,4096], Y f16, f32 accumulate",
                   "l2": "x (33.6 MB) + y (90 MB) + weights (23 MB) per step exceed L2"},
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(tf / peaks["bf16_tflops_sustained"], 4), "traffic": None,
                     "peak_source": f"of {peaks['source']} (sustained)", "kernel": "dq_gemm_kernel<4,false>"},
        "e2e": {"value": round(2.0 * M * N * K * e2e_steps / (ms_e2e * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2},
        "gpu_launches": args.steps, "clocks": cs.summary(),
    }


def run_layer7b(args, torch, sampler_index):
    """Configuration 4: one 7B-shaped decoder layer at decode time (2048 cached rows, the token at position 2048), five
    launches per step; rotation over layer copies (weights + caches 139 MB each) defeats L2."""
    from nnfusion_b200.decoder_layer import DecoderLayer
    from nnfusion_b200.linear import default_context
    H, I, heads, pos, copies = 4096, 11008, 32, 2048, 2
    ctx = default_context(torch.cuda.current_device())
    layers = []
    for _ in range(copies):
        W = [rand_device_weight(torch, n, k) for n, k in ((H, H), (H, H), (H, H), (H, H), (I, H), (I, H), (H, I))]
        g1, g2 = (torch.rand(H, device="cuda") * 0.2 + 0.9 for _ in range(2))
        layer = DecoderLayer(*W, g1, g2, heads=heads, kv_heads=heads, capacity=pos + 1)
        layer.attn.k_cache.normal_()
        layer.attn.v_cache.normal_()
        layers.append(layer)
    x = torch.randn(1, H, device="cuda").to(torch.float16)
    y = torch.empty_like(x)
    ctx.launch_count(reset=True)
    with ClockSampler(sampler_index) as cs:
        ms = timed_graph_steps(torch, [(lambda l=l: l(x, pos, out=y)) for l in layers], args.steps, args.warmup)
    ctx.device_status()
    kv = 2 * heads * pos * 128 * 2
    b = layers[0].weight_bytes + kv + 2 * (3 * H + H + H + 2 * H + I + I + H)
    value = b * args.steps / (ms * 1e-3) / 1e9
    peaks = measured_peaks()
    xh, yh = torch.randn(1, H).to(torch.float16).pin_memory(), torch.empty(1, H, dtype=torch.float16).pin_memory()

    def e2e_step(i):
        x.copy_(xh, non_blocking=True)
        layers[i % copies](x, pos, out=y)
        yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(args.steps, 500)
    ms_e2e = timed_plain_steps(torch, e2e_step, e2e_steps, 3)
    return {
        "metric": "layer7b_decode_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "ms_per_step": ms / args.steps,
        "dtype": "f16", "scaling": "weak",
        "config": {"workload": "layer7b_decode: hidden f16 [1,4096], q/k/v/o u4-g128 [4096,4096], gate/up [11008,4096], "
                               "down [4096,11008], caches f16 2x[32,2049,128], position 2048",
                   "algorithmic_bytes_per_step": b, "launches_per_step": layers[0].launches,
                   "l2": f"rotation over {copies} layers ({copies * b / 1e6:.0f} MB) larger than L2",
                   "launch": "CUDA graph replay of the C-ABI calls"},
        "roofline": {"bound": "hbm", "achieved": round(value, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(value / peaks["hbm_gbs"], 4), "traffic": None,
                     "peak_source": f"of {peaks['source']}", "kernel": "dq_gemv_kernel x4, decode_attention_kernel"},
        "e2e": {"value": round(b * e2e_steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": H * 2, "d2h_bytes_per_step": H * 2},
        "gpu_launches": layers[0].launches * args.steps,
        "clocks": cs.summary(),
    }


def run_mlp70b(args, torch, sampler_index, rank, world, dist):
    """LLaMA-70B-shaped SwiGLU MLP, M = 1 decode, sharded over `world` GPUs.  The shard boundary is closed by the
    one-shot all-reduce kernel over peer memory (launched as a programmatic dependent of the down linear); the same
    step with the sum fused into the down linear's own launch, and with NCCL's all-reduce, is timed beside it."""
    from nnfusion_b200.linear import default_context
    from nnfusion_b200.tp import PeerAllReduce, ShardedMLP, mlp_shapes
    hidden, inter, M = 8192, 28672, 1
    (n_gu, k_gu), (n_d, k_d) = mlp_shapes(hidden, inter, world)
    ctx = default_context(torch.cuda.current_device())
    # per-rank bytes per step must exceed L2 or the weights must rotate
    per_rank = 2 * (linear_bytes(M, n_gu, k_gu) - M * k_gu * 2 - M * n_gu * 2) + linear_bytes(M, n_d, k_d)
    ncopies = max(2, int(L2_BYTES * 2.2 // per_rank) + 1)
    ncopies += ncopies & 1  # an even number of steps per captured graph keeps the all-reduce's two halves in step
    group = dist.group.WORLD if world > 1 else None
    peer = PeerAllReduce(16 * hidden, group) if world > 1 else None
    weights = [(rand_device_weight(torch, n_gu, k_gu), rand_device_weight(torch, n_gu, k_gu),
                rand_device_weight(torch, n_d, k_d)) for _ in range(ncopies)]
    mlps = [ShardedMLP(*w, group=group, reduce="peer" if world > 1 else "nccl", peer=peer) for w in weights]
    x = torch.randn(M, hidden, device="cuda").to(torch.float16)
    ctx.launch_count(reset=True)
    # every captured graph must hold an even number of steps (see PeerAllReduce): K is timed exactly when it is
    # even, K + 1 otherwise, and the line says which
    steps = args.steps + (args.steps & 1)
    # With several ranks the warm-up asks every rank whether one of the exchange's bounded waits gave up; if so the
    # headline is taken with NCCL's all-reduce instead (and says so) rather than from steps that each ran to the limit.
    health = (lambda: ranks_healthy(torch, dist, ctx)) if world > 1 else None
    exchange = "one-shot all-reduce of f16 [1,8192] over peer memory" if world > 1 else "one GPU: no exchange"
    launch = "CUDA graph replay of the C-ABI calls"
    with ClockSampler(sampler_index) as cs:
        try:
            ms = timed_graph_steps(torch, [(lambda m=m: m(x)) for m in mlps], steps, args.warmup,
                                   dist if world > 1 else None, health)
            ctx.device_status()
        except ExchangeUnhealthy as e:
            sys.stderr.write(f"[bench] peer-memory exchange gave up {e}; timing the step with NCCL's all-reduce\n")
            ms = None
    full = 2 * (linear_bytes(M, inter, hidden) - M * hidden * 2 - M * inter * 2) + M * hidden * 2 + 2 * M * inter * 2 + \
        linear_bytes(M, hidden, inter) - M * inter * 2
    peaks = measured_peaks()
    also, nccl, fused_is_headline = {}, None, False
    if world > 1:
        nccl = [ShardedMLP(*w, group=group, reduce="nccl") for w in weights]
        nsteps = min(steps, 400) if ms is not None else steps
        with ClockSampler(sampler_index) as cs_n:
            ms_n = timed_plain_steps(torch, lambda i: nccl[i % ncopies](x), nsteps, max(5, args.warmup), dist)
        if ms is not None:
            also["same_step_with_nccl_allreduce"] = {"us": round(ms_n * 1e3 / nsteps, 2), "launch": "plain launches"}
            also["exchange_as_a_kernel_of_its_own"] = {"us": round(ms * 1e3 / steps, 2), "launch": "CUDA graph replay"}
            fused = [ShardedMLP(*w, group=group, reduce="fused") for w in weights]
            try:
                with ClockSampler(sampler_index) as cs_t:
                    ms_t = timed_graph_steps(torch, [(lambda m=m: m(x)) for m in fused], steps, 4, dist, health)
                ctx.device_status()
                also["exchange_inside_the_down_linear"] = {"us": round(ms_t * 1e3 / steps, 2), "launch": "CUDA graph replay"}
                # both forms of the exchange are this library's kernels over peer memory: the headline is the
                # faster of the two on this box (every rank sees the same two numbers), and says which
                if ms_t < ms:
                    ms, cs, fused_is_headline = ms_t, cs_t, True
                    exchange = ("sum over the ranks inside the down linear's launch (nnf_b200_linear_allreduce), "
                                "f16 [1,8192] over peer memory")
            except ExchangeUnhealthy as e:
                also["exchange_inside_the_down_linear"] = {"us": None, "note": f"a bounded wait gave up {e}"}
        else:
            ms, cs, mlps = ms_n, cs_n, nccl
            exchange, launch = ("NCCL all-reduce of f16 [1,8192] (a bounded wait of the peer-memory exchange gave up "
                                "during the warm-up on this box)"), "plain launches of the C-ABI calls"
    value = full * steps / (ms * 1e-3) / 1e9
    parity = strong = None
    if world > 1:
        using_peer = mlps is not nccl
        parity = mlp_parity(torch, dist, group, rank, world, hidden, inter, peer if using_peer else None)
        # other batch sizes of the configuration at this number of GPUs (the boundary closed by the one-shot kernel
        # up to 16 rows, by NCCL above)
        for m_rows, nsteps in ((16, 200), (256, 60), (4096, 12)):
            xm = torch.randn(m_rows, hidden, device="cuda").to(torch.float16)
            which = mlps if (m_rows <= 16 and using_peer) else nccl
            ms_m = timed_plain_steps(torch, lambda i: which[i % ncopies](xm), nsteps, 4, dist)
            flops = 2.0 * m_rows * 3 * hidden * inter
            also[f"mlp70b_m{m_rows}"] = {"us": round(ms_m * 1e3 / nsteps, 2), "TFLOP/s": round(flops * nsteps / (ms_m * 1e-3) / 1e12, 1),
                                         "exchange": "one-shot kernel" if which is mlps else "NCCL all-reduce",
                                         "launch": "plain launches"}
        # the same workload on ONE of this box's GPUs, timed in this run: what the N-GPU step is measured against
        dist.barrier()
        t1_ms = None
        if rank == 0:
            one = [ShardedMLP(rand_device_weight(torch, inter, hidden), rand_device_weight(torch, inter, hidden),
                              rand_device_weight(torch, hidden, inter)) for _ in range(2)]
            t1_steps = 200
            t1_ms = timed_graph_steps(torch, [(lambda m=m: m(x)) for m in one], t1_steps, 4, repeats=9) / t1_steps
            del one
        dist.barrier()
        if rank == 0:
            tn_ms = ms / steps
            strong = {"t1_us": round(t1_ms * 1e3, 2), "tN_us": round(tn_ms * 1e3, 2), "n": world,
                      "efficiency": round(t1_ms / (world * tn_ms), 4),
                      "note": "t1: the whole MLP (same weights' shapes, same byte count) on rank 0's GPU alone, "
                              "CUDA-graph replay, in this run"}
    xh = torch.randn(M, hidden).to(torch.float16).pin_memory()
    yh = torch.empty(M, hidden, dtype=torch.float16).pin_memory()

    def e2e_step(i):
        x.copy_(xh, non_blocking=True)
        y = mlps[i % ncopies](x)
        yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(steps, 500) // 2 * 2
    ms_e2e = timed_plain_steps(torch, e2e_step, e2e_steps, 4, dist if world > 1 else None)
    ctx.device_status()
    return {
        "metric": "int4_g128_decode_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "steps": steps,
        "ms_per_step": ms / steps, "repeats": REPEATS, "dtype": "f16", "scaling": "strong",
        "config": {"workload": "mlp70b_decode: X f16 [1,8192], gate/up u4-g128 [28672,8192] column-sharded, down [8192,28672] "
                               "row-sharded, " + exchange,
                   "algorithmic_bytes_per_step": full, "parallelism": f"tp{world}",
                   "l2": f"{ncopies} weight copies per rank in rotation ({ncopies * per_rank / 1e6:.0f} MB per rank) larger than L2",
                   "launch": launch},
        "roofline": {"bound": "hbm", "achieved": round(value / world, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(value / world / peaks["hbm_gbs"], 4), "traffic": None,
                     "traffic_note": "not captured: ncu runs on one rank of one GPU only, and a rank's kernels wait for "
                                     "its peers; the one-GPU captures show traffic = algorithmic bytes for this kernel",
                     "peak_source": f"of {peaks['source']}, per GPU",
                     "kernel": "dq_gemv_direct_kernel (gate/up fused SiLU*mul, down)"},
        **({"parity": parity} if parity else {}),
        **({"strong_scaling": strong} if strong else {}),
        "e2e": {"value": round(full * e2e_steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": M * hidden * 2, "d2h_bytes_per_step": M * hidden * 2},
        # gate/up, down and (as a kernel of its own) the exchange; NCCL's kernel is not counted
        "gpu_launches": (3 if (world > 1 and mlps is not nccl and not fused_is_headline) else 2) * steps,
        "clocks": cs.summary(),
        **({"also": also} if also else {}),
    }


def mlp_parity(torch, dist, group, rank, world, hidden, inter, peer):
    """One step of the sharded MLP on seeded weights against the same MLP on one GPU (rank 0 computes it, everybody
    compares), for M = 1 and 16, plus bit-equality of the ranks' results.  Returns what the bench line prints."""
    from nnfusion_b200.tp import ShardedMLP
    g, u, d = (rand_device_weight(torch, n, k, seed=s) for n, k, s in
               ((inter, hidden, 101), (inter, hidden, 102), (hidden, inter, 103)))
    sharded = ShardedMLP(g.shard_rows(rank, world), u.shard_rows(rank, world), d.shard_k(rank, world), group=group,
                         reduce="peer" if peer is not None else "nccl", peer=peer)
    whole = ShardedMLP(g, u, d) if rank == 0 else None
    worst, identical = 0.0, True
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    for m_rows in (1, 16):
        x = torch.randn(m_rows, hidden, device="cuda", generator=gen).to(torch.float16)
        # two calls: the exchange's two buffer halves stay in step with every other user of the same buffers
        y = sharded(x).clone()
        y2 = sharded(x)
        ref = whole(x).clone() if rank == 0 else torch.empty_like(y)
        dist.broadcast(ref, 0, group=group)
        err = (y.float() - ref.float()).abs().max() / ref.float().abs().max()
        t = torch.stack([err, (y != y2).any().float()])
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        worst = max(worst, float(t[0]))
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y, group=group)
        identical = identical and float(t[1]) == 0.0 and all(bool((ys[0] == o).all()) for o in ys[1:])
    torch.cuda.synchronize()
    return {"max_rel_err_vs_one_gpu": worst, "tolerance": 5e-3, "within_tolerance": worst <= 5e-3,
            "ranks_bit_identical": identical, "rows": [1, 16],
            "how": "seeded weights, the sharded step against the unsharded MLP on rank 0's GPU, max|y-r|/max|r|"}


# ----------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="auto", choices=["auto", "decode_gemv", "mlp70b_decode", "prefill_gemm", "layer7b_decode", "config1_gemv"])
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary measurements at 1 GPU")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    workload = args.workload
    if workload == "auto":
        workload = "decode_gemv" if max(world, args.gpus) == 1 else "mlp70b_decode"

    # torch.distributed.run sets OMP_NUM_THREADS=1 for its workers when the variable is unset.  The CPU baseline (the
    # reference arm's one working rank; rank 0 of a one-GPU run) is meant to use every host core, so that default is
    # undone before anything loads OpenMP.
    if (rank == 0 and (args.impl == "reference" or world == 1) and "TORCHELASTIC_RUN_ID" in os.environ
            and os.environ.get("OMP_NUM_THREADS") == "1"):
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))

    if args.impl == "reference":
        # The reference's CPU path, rank 0 only; other ranks leave without work.
        if rank != 0:
            return 0
        steps = args.steps if args.steps is not None else 20
        warmup = args.warmup if args.warmup is not None else 3
        if workload == "prefill_gemm":
            M, K, rows, full_rows = 4096, 4096, 344, 11008
        elif workload == "mlp70b_decode":
            M, K, rows, full_rows = 1, 8192, 896, 28672
        else:
            M, K, rows, full_rows = 1, 4096, 1376, 11008
        sec, n, cores, kind = cpu_reference_gemv(0.0, rows, K, M, steps=steps, warmup=warmup)
        if workload == "prefill_gemm":
            value, unit, metric = 2.0 * M * rows * K / sec / 1e12, "TFLOP/s", "int4_g128_prefill_gemm_tflops"
        else:
            value, unit, metric = linear_bytes(M, rows, K) / sec / 1e9, "GB/s", "int4_g128_decode_gemv_hbm_gbs"
        sample = (f"{rows} of {full_rows} weight rows per step (same K, same M); Convert/Subtract/Multiply restated, "
                  f"Dot = reference MLAS SGEMM" if kind == "reference" else f"{rows} of {full_rows} rows, C restatement")
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": n,
            "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong" if workload == "mlp70b_decode" else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload + " (CPU reference path)"},
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return 0

    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path for --impl ours"}))
        return 2
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if workload == "decode_gemv":
            steps_default, warmup_default = 2400, 240
        elif workload == "prefill_gemm":
            steps_default, warmup_default = 50, 5
        else:
            steps_default, warmup_default = 400, 40
        args.steps = args.steps if args.steps is not None else steps_default
        args.warmup = max(3, args.warmup if args.warmup is not None else warmup_default)

        if workload == "decode_gemv":
            out, *_ = run_decode_gemv(args, torch, local_rank)
        elif workload == "prefill_gemm":
            out = run_prefill_gemm(args, torch, local_rank)
        elif workload == "layer7b_decode":
            out = run_layer7b(args, torch, local_rank)
        elif workload == "config1_gemv":
            out = run_config1_gemv(args, torch, local_rank)
        else:
            out = run_mlp70b(args, torch, local_rank, rank, world, dist)
        if rank == 0:
            out.setdefault("steps", args.steps)
            out.update({"n_gpus": world, "warmup": args.warmup, "higher_is_better": True,
                        "vs_baseline": None, "data": "synthetic", "impl": "ours"})
            if world == 1:
                # the reference's CPU path on this box's host cores, bounded sample
                if workload == "prefill_gemm":
                    sec, n, cores, kind = cpu_reference_gemv(10.0, 344, 4096, 4096)
                    v, unit = 2.0 * 4096 * 344 * 4096 / sec / 1e12, "TFLOP/s"
                    sample = "344 of 11008 weight rows, M = 4096, ~10 s"
                elif workload == "config1_gemv":
                    sec, n, cores, kind = cpu_reference_gemv(10.0, 512, 4096, 16)
                    v, unit = linear_bytes(16, 512, 4096, bits=8, group=4096, act_bytes=4, scale_bytes=4) / sec / 1e9, "GB/s"
                    sample = ("512 of 4096 weight rows, M = 16 (the dequant graph on group-128 uint4 test data: the "
                              "element-wise kernels and the SGEMM see the same fp32 sizes), ~10 s of calls")
                elif workload == "mlp70b_decode":
                    sec, n, cores, kind = cpu_reference_gemv(10.0, 896, 8192, 1)
                    v, unit = linear_bytes(1, 896, 8192) / sec / 1e9, "GB/s"
                    sample = "896 of 28672 gate rows (K = 8192), ~10 s"
                else:
                    sec, n, cores, kind = cpu_reference_gemv(10.0, 1376, 4096, 1)
                    v, unit = linear_bytes(1, 1376, 4096) / sec / 1e9, "GB/s"
                    sample = "1376 of 11008 weight rows per call (dequant graph + MLAS SGEMM), ~10 s of calls"
                out["cpu_baseline"] = {"value": v, "unit": unit, "cores": cores, "kind": kind, "sample": sample,
                                       "calls": n, "ms_per_call": sec * 1e3}
                if workload == "decode_gemv":
                    g = cpu_reference_gemm_only(1376, 4096, 1)
                    if g is not None:
                        out["cpu_baseline"]["gemm_only_on_dequantised_fp32_ms_per_call"] = g * 1e3
                if not args.no_extras:
                    out["also"] = extra_measurements(torch)
            order = ["metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                     "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks"]
            line = {k: out[k] for k in order if k in out}
            line.update({k: v for k, v in out.items() if k not in line})
            print(json.dumps(line))
    finally:
        if dist is not None:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
