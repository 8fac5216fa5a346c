#!/usr/bin/env python
"""Benchmark of the NVFP4 linear path on B200 (headline), with legs for the attention kernels and RoPE.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--profile-case NAME]

N = 1 (default): the square single-GPU GEMM the headline metric is quoted on (M = N = K = 4096,
activations N(0,1) with 0.5 % x30 outliers, weights N(0,0.02), both quantised to NVFP4).  One
step = one `linear()` call on operands already resident in HBM; `value` is 2*M*N*K / step time
in TFLOP/s.  The same run also measures the quantiser bandwidth on bf16 [32768, 8192], the
end-to-end number (host buffers -> H2D -> quantize -> linear -> D2H) and the CPU emulation.

N > 1 (launched with torchrun): the column-parallel MLP up/gate GEMM (M = 8192, K = 8192,
N = 28672 split over the ranks) followed by the NCCL all-gather of the bf16 output; total work
is fixed, so "scaling" is "strong".

`--impl reference` times the reference's CPU-runnable form of this path (the torch emulation its
own tests use as the oracle: dequantise -> fp32 matmul -> cast) on the host cores.

Rank 0 prints exactly one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
NOMINAL_FP4_TFLOPS = 9000.0     # dense FP4, vendor figure
NOMINAL_HBM_GBS = 8000.0
METRIC = "NVFP4 GEMM TFLOP/s at 4096^3 (% of FP4 peak); quantize HBM GB/s (% of 8 TB/s)"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------
# clock sampling through NVML while the timed region runs
# ------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples = []
        self.stop = threading.Event()
        self.thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and vis.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self.stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        if self.thread is not None:
            self.thread.join()

    def summary(self, t0=None, t1=None):
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0,
                    "note": "NVML unavailable"}
        window = "timed"
        sel = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1]
        if len(sel) < 3:
            sel, window = self.samples, "warmup+timed"
        mhz = sorted(s[1] for s in sel)
        bits = 0
        for s in sel:
            bits |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if bits & bit]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(sel), "window": window}


# ------------------------------------------------------------------------------------------
# synthetic inputs
# ------------------------------------------------------------------------------------------
def activations(shape, seed, frac, mul, device):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(shape, generator=g, device=device)
    if frac > 0:
        mask = torch.rand(shape, generator=g, device=device) < frac
        x = torch.where(mask, x * mul, x)
    return x.bfloat16()


def weights(shape, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device) * 0.02).bfloat16()


def time_graph(fn_step, n_sets, steps, warmup, barrier=None):
    """Capture `steps` calls of fn_step(i % n_sets) in a CUDA graph and time one replay with
    events (launch overhead of the Python wrapper would otherwise dominate 20-microsecond
    kernels).  Returns (seconds for the K steps, host t0, host t1)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for i in range(max(warmup, 3)):
            fn_step(i % n_sets)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(steps):
            fn_step(i % n_sets)
    graph.replay()                      # one untimed replay: graph upload, caches
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    time_graph.last_graph = graph
    return e0.elapsed_time(e1) * 1e-3, t0, t1


def sustained_run(graph, steps_per_replay, flops_per_step, device_index, seconds=2.5):
    """Replay `graph` back to back for `seconds`, CUDA events around the whole run, NVML clock samples
    inside it: what the kernel does once the power cap has set the clock."""
    torch.cuda.synchronize()
    one = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    one[0].record()
    graph.replay()
    one[1].record()
    torch.cuda.synchronize()
    replays = max(10, int(seconds / max(one[0].elapsed_time(one[1]) * 1e-3, 1e-6)))
    with ClockSampler(device_index) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    secs = e0.elapsed_time(e1) * 1e-3
    c = clk.summary(t0, t1)
    tflops = flops_per_step * steps_per_replay * replays / secs / 1e12
    ghz = (c["sm_mhz"] or 0) / 1e3
    return {"value": tflops, "unit": "TFLOP/s", "seconds": secs, "launches": steps_per_replay * replays,
            "us_per_step": secs / (steps_per_replay * replays) * 1e6, "clock_samples": c["samples"],
            "sm_mhz_median": c["sm_mhz"], "sm_max_mhz": c["sm_max_mhz"], "reasons": c["reasons"],
            "tflops_per_ghz": tflops / ghz if ghz else None}


def time_eager(fn, reps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


# ------------------------------------------------------------------------------------------
# CPU emulation (the reference's CPU-runnable form of the path)
# ------------------------------------------------------------------------------------------
def cpu_emulation_c2(budget_s=15.0, reps=None):
    """dequantise -> fp32 matmul -> bf16 on the whole 4096^3 workload, all host threads, as many repetitions
    as fit the budget.  Returns (TFLOP/s, cores, sample description, seconds per rep, reps)."""
    from oracle import emulation as emu
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = k = 4096
    g = torch.Generator().manual_seed(0)
    w = (torch.randn((n, k), generator=g) * 0.02).bfloat16()
    w4, wsf, wg = emu.quantize_nvfp4_ref(w)
    rows = 4096
    a = torch.randn((rows, k), generator=g).bfloat16()
    a4, asf, ag = emu.quantize_nvfp4_ref(a)
    t = time.perf_counter()
    emu.linear_nvfp4_ref(a4, asf, ag, w4, wsf, wg)
    first = time.perf_counter() - t
    if reps is None:
        reps = max(1, min(10, int(budget_s / max(first, 1e-3))))
    t = time.perf_counter()
    for _ in range(reps):
        emu.linear_nvfp4_ref(a4, asf, ag, w4, wsf, wg)
    dt = (time.perf_counter() - t) / reps
    tflops = 2.0 * rows * n * k / dt / 1e12
    sample = f"the whole 4096^3 configuration, dequantise + fp32 matmul + cast, {reps} repetitions"
    return tflops, cores, sample, dt, reps


C2_WORKLOAD = ("single-GPU square NVFP4 GEMM M=N=K=4096, activations N(0,1) + 0.5% x30 outliers, "
               "weights N(0,0.02), 128x4 scale tiles, bf16 out, alpha = gA*gB")


def c5_workload(world):
    return (f"column-parallel NVFP4 GEMM M=8192 K=8192 N=28672 over {world} GPUs "
            f"(N/{world} = {28672 // world} columns per rank) + all-gather of the bf16 output "
            "(fused into the GEMM epilogue: TMA stores to every rank's buffer over NVLink)")


def run_reference(args):
    """The reference's CPU-runnable form of the path (its tests' torch emulation: dequantise -> fp32 matmul ->
    cast, restated in oracle/emulation.py) on the host cores.  N = 1: the whole 4096^3 configuration, every
    step.  N > 1: the column-parallel configuration is 28 times larger (3.85 TFLOP per step, about 10 s per
    step on 16 cores), so a step is a sample: 512 of the 8192 activation rows against 4096 of the 28672 weight
    rows, K in full, with the weight dequantised once outside the timed loop as a serving stack would."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    warmup = max(args.warmup, 3)
    from oracle import emulation as emu
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    if args.gpus > 1:
        n, k, rows = 4096, 8192, 512
        workload = c5_workload(args.gpus)
        what = (f"{rows} of 8192 activation rows x {n} of 28672 weight rows (K = 8192 in full), weight dequantised "
                "outside the timed loop")
        scaling = "strong"
        w = (torch.randn((n, k), generator=g) * 0.02).bfloat16()
        w4, wsf, wg = emu.quantize_nvfp4_ref(w, sf_layout="128x4")
        wd = emu.dequantize_nvfp4_ref(w4, wsf, None)
        a = torch.randn((rows, k), generator=g).bfloat16()
        a4, asf, ag = emu.quantize_nvfp4_ref(a, sf_layout="128x4")

        def step():
            ad = emu.dequantize_nvfp4_ref(a4, asf, None)
            return ((ad @ wd.t()) * (ag * wg)).to(torch.bfloat16)
    else:
        n = k = rows = 4096
        workload = C2_WORKLOAD
        what = "the whole configuration: 4096 activation rows x 4096 x 4096 weight, dequantise + fp32 matmul + cast"
        scaling = "weak"
        w = (torch.randn((n, k), generator=g) * 0.02).bfloat16()
        w4, wsf, wg = emu.quantize_nvfp4_ref(w, sf_layout="128x4")
        a = torch.randn((rows, k), generator=g)
        a = torch.where(torch.rand((rows, k), generator=g) < 0.005, a * 30.0, a).bfloat16()
        a4, asf, ag = emu.quantize_nvfp4_ref(a, sf_layout="128x4")

        def step():
            return emu.linear_nvfp4_ref(a4, asf, ag, w4, wsf, wg)
    for _ in range(warmup):
        step()
    t = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t > 150:
            break
    dt = (time.perf_counter() - t) / done
    tflops = 2.0 * rows * n * k / dt / 1e12
    sample = f"each step = {what}; {done} steps timed on {cores} host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": done, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's GEMM kernel is sm_120a-only and cannot run on a B200; its CPU-runnable "
                "form is the torch emulation from its tests, restated in oracle/emulation.py",
    }
    gpu_side = reference_gpu_kernels() if args.gpus == 1 else None
    if gpu_side is not None:
        line["reference_gpu_kernels"] = gpu_side
    print(json.dumps(line))


def reference_gpu_kernels():
    """The part of the reference that does run on a B200: its own quantiser kernels (oracle/_ref, built unchanged
    from the reference checkout for sm_100a), timed on the quantiser configuration of the benchmark, bf16
    [32768, 8192].  None without a GPU or without that build."""
    if not torch.cuda.is_available():
        return None
    from oracle import build_ref
    ref = build_ref.load()
    if ref is None:
        return None
    m, k = 32768, 8192
    x = torch.randn((m, k), dtype=torch.bfloat16, device="cuda")
    gs = (x.abs().max().float() / (6.0 * 448.0)).reshape(())
    out4 = torch.empty((m, k // 2), dtype=torch.uint8, device="cuda")
    sf4 = torch.empty((k // 64, m, 4), dtype=torch.float8_e4m3fn, device="cuda")
    out8 = torch.empty((m, k), dtype=torch.float8_e4m3fn, device="cuda")
    outi = torch.empty((m, k), dtype=torch.int8, device="cuda")
    sf8 = torch.empty((m,), dtype=torch.float32, device="cuda")
    smax_f = torch.tensor(448.0, device="cuda")
    smax_i = torch.tensor(127, dtype=torch.int32, device="cuda")

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e-3

    t4 = timed(lambda: ref.quantize_nvfp4(out4, sf4, x, gs, 0, 1, False))
    t8 = timed(lambda: ref.quantize_fp8(out8, sf8, x, smax_f, 0, 1, False))
    ti = timed(lambda: ref.quantize_int8(outi, sf8, x, smax_i, 0, 1))
    b4 = x.numel() * 2 + out4.numel() + sf4.numel()
    b8 = x.numel() * 3 + sf8.numel() * 4
    return {"workload": "bf16 [32768, 8192], the reference's own kernels compiled for sm_100a, inputs larger than L2",
            "quantize_nvfp4_gbs": b4 / t4 / 1e9, "quantize_nvfp4_us": t4 * 1e6,
            "quantize_fp8_gbs": b8 / t8 / 1e9, "quantize_int8_gbs": b8 / ti / 1e9,
            "note": "given the global scale; compare with the `quantize` record of the other arm"}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def quantize_bandwidth(peaks):
    """BASELINE config 4: bf16 [32768, 8192] with 1 % x50 outliers."""
    from ac4k_kernel_b200 import _cuda_ops, ops
    from ac4k_kernel_b200.ops.quant import _global_scale
    m, k = 32768, 8192
    x = activations((m, k), 0, 0.01, 50.0, "cuda")
    g = _global_scale(x, 2688.0)
    out = torch.empty((m, k // 2), dtype=torch.uint8, device="cuda")
    res = {}
    for name, shape in (("ac4k", (k // 64, m, 4)), ("128x4", (m // 128, k // 64, 32, 4, 4))):
        sf = torch.empty(shape, dtype=torch.float8_e4m3fn, device="cuda")
        t = time_eager(lambda: _cuda_ops.quantize_nvfp4(out, sf, x, g, 0, 1, False), 20)
        res[f"nvfp4_{name}_gbs"] = m * k * 2.5625 / t / 1e9
    t = time_eager(lambda: _global_scale(x, 2688.0), 20)
    res["global_scale_gbs"] = m * k * 2 / t / 1e9
    t = time_eager(lambda: ops.quantize(x, 0, 1), 10)
    res["quantize_call_us"] = t * 1e6
    for prec in ("fp8e4m3", "int8"):
        t = time_eager(lambda: ops.quantize(x, 0, 1, precision=prec), 10)
        res[f"{prec}_gbs"] = (m * k * 3 + m * 4) / t / 1e9
    best = max(res["nvfp4_ac4k_gbs"], res["nvfp4_128x4_gbs"])
    res["nvfp4_frac_of_8tbs"] = best / NOMINAL_HBM_GBS
    res["nvfp4_frac_of_measured_copy"] = best / peaks["hbm_gbs"]
    res["workload"] = "bf16 [32768, 8192] N(0,1) with 1% x50 outliers; 688 MB per launch (larger than L2)"
    return res


def decode_stream(peaks):
    """BASELINE config 3: M in {1, 16, 64}, N = K = 8192, weights quantised once; 8 weight copies are
    rotated (8 x 37.7 MB > 2 x L2) and 40 calls are replayed from one CUDA graph."""
    from ac4k_kernel_b200 import _cuda_ops, ops
    n = k = 8192
    w = weights((n, k), 1, "cuda")
    w4, wsf, wg = ops.quantize(w, 0, 1, sf_layout="128x4")
    del w
    sets = [(w4.clone(), wsf.clone()) for _ in range(8)]
    stream_bytes = n * k // 2 + n * k // 16
    res = {"workload": "decode GEMM M x 8192 x 8192 against resident NVFP4 weights, 8 weight copies rotated",
           "algorithmic_bytes_per_call": stream_bytes}
    for m in (1, 16, 64):
        a = activations((m, k), 2, 0.0, 1.0, "cuda")
        a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

        def step(i):
            _cuda_ops.linear_nvfp4(out, a4, asf, ag, sets[i][0], sets[i][1], wg, None)

        secs, _, _ = time_graph(step, 8, 40, 3)
        t = secs / 40
        res[f"m{m}_us"] = t * 1e6
        res[f"m{m}_weight_gbs"] = stream_bytes / t / 1e9
    res["m16_frac_of_8tbs"] = res["m16_weight_gbs"] / NOMINAL_HBM_GBS
    res["m16_frac_of_measured_copy"] = res["m16_weight_gbs"] / peaks["hbm_gbs"]
    return res


def attention_nvfp4(peaks):
    """Both attention precisions at the shape of the reference's test/test_attention_tflops.py:36-39 ([1, 75600, 40, 128];
    its flop count 4 B H N^2 D, :32; it times `attention(precision="int8+fp8e4m3")`, quantisers included) and a shorter
    one: the kernels alone on resident quantised operands, the `attention()` calls with their quantiser launches, and
    torch's bf16 scaled_dot_product_attention on the same tensors as a library yardstick."""
    import math
    import torch.nn.functional as F
    from ac4k_kernel_b200 import _cuda_ops, ops
    from ac4k_kernel_b200.ops.attention import _int8_quantize
    res = {"unit": "TFLOP/s", "flops": "4 * B * H * N^2 * D", "cases": []}
    for (b, n, h, d, reps) in ((1, 16384, 16, 128, 10), (1, 75600, 40, 128, 3)):
        g = torch.Generator(device="cuda").manual_seed(9567)
        q, k, v = (torch.randn((b, n, h, d), dtype=torch.bfloat16, device="cuda", generator=g) for _ in range(3))
        out = torch.empty_like(q)
        view = out.permute(0, 2, 1, 3)
        flops = 4.0 * b * h * n * n * d
        case = {"shape_BNHD": [b, n, h, d]}
        qq, qs, qg = ops.quantize(q, 1, 3, sf_layout="128x4")
        kq, ks, kg = ops.quantize(k, 1, 3, sf_layout="128x4")
        vq, vs, vg = ops.quantize(v, 3, 1, swizzle=True, sf_layout="128x4")
        t_k = time_eager(lambda: _cuda_ops.mha_nvfp4_fwd(view, qq, qs, qg, kq, ks, kg, vq, vs, vg, 1 / math.sqrt(d)), reps)
        t_a = time_eager(lambda: ops.attention(q, k, v, layout="BNHD", precision="nvfp4", out=out), reps)
        case.update({"kernel_ms": t_k * 1e3, "kernel_tflops": flops / t_k / 1e12,
                     "attention_call_ms": t_a * 1e3, "attention_call_tflops": flops / t_a / 1e12})
        del qq, kq, vq
        q8, q8s = _int8_quantize(q, "BNHD", 1, BLOCK_SIZE=64)
        k8, k8s = _int8_quantize(k, "BNHD", 1, BLOCK_SIZE=128)
        v8, v8s = ops.quantize(v, 3, 1, swizzle=True, max_scale=2.25, precision="fp8e4m3")
        t_k8 = time_eager(lambda: _cuda_ops.mha_int8_x_fp8_fwd(view, q8, q8s, 64, k8, k8s, 128, v8, v8s, 1 / math.sqrt(d)), reps)
        t_a8 = time_eager(lambda: ops.attention(q, k, v, layout="BNHD", precision="int8+fp8e4m3", out=out), reps)
        case.update({"int8_x_fp8_kernel_ms": t_k8 * 1e3, "int8_x_fp8_kernel_tflops": flops / t_k8 / 1e12,
                     "int8_x_fp8_attention_call_ms": t_a8 * 1e3, "int8_x_fp8_attention_call_tflops": flops / t_a8 / 1e12})
        del q8, k8, v8
        t_s = time_eager(lambda: F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)), reps)
        case.update({"torch_sdpa_bf16_ms": t_s * 1e3, "torch_sdpa_bf16_tflops": flops / t_s / 1e12})
        res["cases"].append(case)
        del q, k, v, out
    res["note"] = ("both kernels are bounded by the softmax (16 ex2 per clock per SM = 1024 cycles per 128 x 128 scores), not by "
                   "the four- or eight-bit MMAs; inputs are larger than L2 at both shapes")
    return res


def rope3d_stream(peaks):
    """3-D rotary embedding at the shape of the reference's test (test/test_rope_3d_apply.py:49-56): [1, 21 * 45 * 80,
    40, 128] bf16 with a 1024-row complex128 table; 2 bytes read + 2 written per element, 1.55 GB per launch."""
    from ac4k_kernel_b200 import ops
    f, h, w, n, d = 21, 45, 80, 40, 128
    g = torch.Generator(device="cuda").manual_seed(9567)
    x = torch.randn((1, f * h * w, n, d), dtype=torch.bfloat16, device="cuda", generator=g)
    grid = torch.tensor([[f, h, w]], dtype=torch.int32, device="cuda")
    ang = torch.outer(torch.arange(1024, dtype=torch.float64),
                      1.0 / torch.pow(torch.tensor(10000.0, dtype=torch.float64), torch.arange(0, d, 2, dtype=torch.float64) / d))
    freqs = torch.polar(torch.ones_like(ang), ang).cuda()
    out = torch.empty_like(x)
    t = time_eager(lambda: ops.rope3d(x, grid, freqs, out), 10)
    gbs = x.numel() * 4 / t / 1e9
    return {"workload": "rope3d bf16 [1, 75600, 40, 128], grid 21 x 45 x 80, complex128 table [1024, 64]",
            "ms": t * 1e3, "gbs": gbs, "frac_of_8tbs": gbs / NOMINAL_HBM_GBS, "frac_of_measured_copy": gbs / peaks["hbm_gbs"],
            "algorithmic_bytes_per_launch": x.numel() * 4}


def c5_single_gpu():
    """BASELINE config 5 on one GPU (M = K = 8192, N = 28672): the same-workload base of the 1 -> N curve.
    One operand set (600 MB, larger than L2), 5 steps in a graph."""
    from ac4k_kernel_b200 import _cuda_ops, ops
    m, k, n = 8192, 8192, 28672
    a = activations((m, k), 0, 0.005, 30.0, "cuda")
    w = weights((n, k), 1000, "cuda")
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    w4, wsf, wg = ops.quantize(w, 0, 1, sf_layout="128x4")
    del a, w
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

    def step(i):
        _cuda_ops.linear_nvfp4(out, a4, asf, ag, w4, wsf, wg, None)

    steps = 5
    secs, _, _ = time_graph(step, 1, steps, 3)
    t = secs / steps
    return {"workload": "NVFP4 GEMM M=8192 K=8192 N=28672 on one GPU (no exchange)", "ms_per_step": t * 1e3,
            "value": 2.0 * m * n * k / t / 1e12, "unit": "TFLOP/s", "steps": steps,
            "frac_of_nominal_fp4_peak": 2.0 * m * n * k / t / 1e12 / NOMINAL_FP4_TFLOPS}


def run_single(args, peaks):
    from ac4k_kernel_b200 import _cuda_ops, ops
    torch.cuda.set_device(0)
    m = n = k = 4096
    flops = 2.0 * m * n * k
    a = activations((m, k), 0, 0.005, 30.0, "cuda")
    w = weights((n, k), 1, "cuda")
    set_bytes = m * k // 2 + n * k // 2 + (m + n) * k // 16 + m * n * 2
    n_sets = 2 * L2_BYTES // set_bytes + 1          # rotate operand sets: > 2 x L2 in total
    sets = {}
    for layout in ("128x4", "ac4k"):
        a4, asf, ag = ops.quantize(a, 0, 1, sf_layout=layout)
        w4, wsf, wg = ops.quantize(w, 0, 1, sf_layout=layout)
        sets[layout] = [(a4.clone(), asf.clone(), ag, w4.clone(), wsf.clone(), wg,
                         torch.empty((m, n), dtype=torch.bfloat16, device="cuda")) for _ in range(n_sets)]

    def step(layout):
        def f(i):
            a4, asf, ag, w4, wsf, wg, out = sets[layout][i]
            _cuda_ops.linear_nvfp4(out, a4, asf, ag, w4, wsf, wg, None)
        return f

    with ClockSampler(0) as clk:
        secs, t0, t1 = time_graph(step("128x4"), n_sets, args.steps, args.warmup)
    clocks = clk.summary(t0, t1)
    main_graph = time_graph.last_graph
    # the reference's scale layout next, under the same (burst) conditions as the headline value
    secs_ac4k, _, _ = time_graph(step("ac4k"), n_sets, args.steps, args.warmup)
    # the same graph replayed back to back for seconds: throughput at the clock the power cap settles on
    sustained = sustained_run(main_graph, args.steps, flops, 0)
    if peaks.get("bf16_tflops_sustained"):
        sustained["frac_of_4x_measured_bf16_sustained"] = sustained["value"] / (4.0 * peaks["bf16_tflops_sustained"])
    sustained["frac_of_nominal_fp4_peak"] = sustained["value"] / NOMINAL_FP4_TFLOPS
    ms_per_step = secs / args.steps * 1e3
    value = flops / (secs / args.steps) / 1e12
    del sets["ac4k"]

    # end to end through the public API with host buffers: H2D of the step's activations,
    # quantize (global scale + quantiser), linear against resident NVFP4 weights, D2H of the result
    # The steps are software-pipelined over three buffers and three streams (the copy engines run
    # both directions at once): H2D of step i+1, compute of step i and D2H of step i-1 overlap, every
    # step's own copies stay inside the timed region.
    a_host = a.cpu().pin_memory()
    _, _, _, w4, wsf, wg, _ = sets["128x4"][0]
    nbuf = 3
    out_hosts = [torch.empty((m, n), dtype=torch.bfloat16).pin_memory() for _ in range(nbuf)]
    a_devs = [torch.empty_like(a) for _ in range(nbuf)]
    out_devs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in range(nbuf)]
    s_h2d, s_d2h = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    ev_h2d = [torch.cuda.Event() for _ in range(nbuf)]
    ev_comp = [torch.cuda.Event() for _ in range(nbuf)]
    ev_d2h = [torch.cuda.Event() for _ in range(nbuf)]

    def e2e_step(i):
        b = i % nbuf
        with torch.cuda.stream(s_h2d):
            if i >= nbuf:
                s_h2d.wait_event(ev_comp[b])          # the step that last read a_devs[b] is done
            a_devs[b].copy_(a_host, non_blocking=True)
            ev_h2d[b].record(s_h2d)
        main.wait_event(ev_h2d[b])
        if i >= nbuf:
            main.wait_event(ev_d2h[b])                # out_devs[b] has been copied out
        a4, asf, ag = ops.quantize(a_devs[b], 0, 1, sf_layout="128x4")
        ops.linear(a4, asf, ag, w4, wsf, wg, out=out_devs[b])
        ev_comp[b].record(main)
        with torch.cuda.stream(s_d2h):
            s_d2h.wait_event(ev_comp[b])
            out_hosts[b].copy_(out_devs[b], non_blocking=True)
            ev_d2h[b].record(s_d2h)

    def e2e_run(reps):
        for i in range(reps):
            e2e_step(i)
        main.wait_stream(s_h2d)
        main.wait_stream(s_d2h)

    e2e_reps = max(6, min(args.steps, 60))
    e2e_run(6)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_reps)
    e1.record()
    torch.cuda.synchronize()
    t_e2e = e0.elapsed_time(e1) * 1e-3 / e2e_reps
    # the result that came back is the GEMM's: compare the last step's host copy with a device-side run
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    check = ops.linear(a4, asf, ag, w4, wsf, wg)
    e2e_ok = bool(torch.equal(out_hosts[(e2e_reps - 1) % nbuf], check.cpu()))
    e2e = {"value": flops / t_e2e / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": a_host.numel() * 2,
           "d2h_bytes_per_step": out_hosts[0].numel() * 2, "ms_per_step": t_e2e * 1e3,
           "result_matches_device_run": e2e_ok,
           "path": "pinned host bf16 activations -> H2D -> quantize() -> linear() vs resident NVFP4 weights -> "
                   "D2H of bf16 output; steps pipelined over 3 buffers / 3 streams"}
    del out_hosts, a_devs, out_devs
    del sets, a_host

    c5 = c5_single_gpu()
    quant = quantize_bandwidth(peaks)
    decode = decode_stream(peaks)
    attn = attention_nvfp4(peaks)
    rope = rope3d_stream(peaks)
    cpu_tflops, cores, sample, _, _ = cpu_emulation_c2()

    fp4_proxy_peak = 4.0 * peaks["bf16_tflops"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": C2_WORKLOAD,
                   "l2": f"{n_sets} operand/output sets rotated ({n_sets * set_bytes >> 20} MiB > 2 x L2)",
                   "timing": "K steps captured in one CUDA graph, CUDA events around the replay"},
        "frac_of_nominal_fp4_peak": value / NOMINAL_FP4_TFLOPS,
        "tflops_per_ghz": value / (clocks["sm_mhz"] / 1e3) if clocks.get("sm_mhz") else None,
        "sustained": sustained,
        "c5_single_gpu": c5,
        "value_reference_scale_layout": flops / (secs_ac4k / args.steps) / 1e12,
        "roofline": {"bound": "tensor", "achieved": value, "peak": fp4_proxy_peak, "unit": "TFLOP/s",
                     "frac": value / fp4_proxy_peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum per launch is not measured inside this run (it
                     # needs ncu); the figure of the capture of one launch is in the file named here
                     "traffic": None, "traffic_source": "profiles/gemm_nvfp4_pair_4096cube.md",
                     "peak_note": f"4 x {peaks['source']} bf16 burst ({peaks['bf16_tflops']} TFLOP/s): no FP4 figure is "
                                  "measured on this pool; nominal dense FP4 is 9000 TFLOP/s",
                     "algorithmic_flops_per_launch": flops},
        "quantize": quant,
        "decode": decode,
        "attention_nvfp4": attn,
        "rope3d": rope,
        "cpu_baseline": {"value": cpu_tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": e2e,
        "clocks": clocks,
        "gpu_launches": args.steps,
    }
    print(json.dumps(line))


def run_multi(args, peaks):
    import torch.distributed as dist
    from ac4k_kernel_b200 import ops, parallel, _cuda_ops
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    # a rank that fails must not leave the others waiting for long: collectives give up after 3 minutes
    import datetime
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    m, k, n = 8192, 8192, 28672
    flops = 2.0 * m * n * k
    lo, hi = parallel.shard_bounds(n, rank, world)
    ns = hi - lo
    a = activations((m, k), 0, 0.005, 30.0, "cuda")          # replicated: same seed on every rank
    # this rank's rows of the weight, drawn from a per-shard seed (the full matrix is never built)
    w_shard = weights((ns, k), 1000 + rank, "cuda")
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    w4, wsf, wg = parallel.quantize_weight_shard(w_shard, None, "128x4")
    del a, w_shard
    set_bytes = ns * k // 2 + ns * k // 16 + m * ns * 2
    n_sets = max(2, 2 * L2_BYTES // set_bytes + 1)
    wsets = [(w4.clone(), wsf.clone(), torch.empty((m, ns), dtype=torch.bfloat16, device="cuda"))
             for _ in range(n_sets)]
    gathered = torch.empty((world, m, ns), dtype=torch.bfloat16, device="cuda")

    def gemm_only(i):
        wq, ws, out = wsets[i]
        _cuda_ops.linear_nvfp4(out, a4, asf, ag, wq, ws, wg, None)

    def full_step(i):
        wq, ws, out = wsets[i]
        _cuda_ops.linear_nvfp4(out, a4, asf, ag, wq, ws, wg, None)
        dist.all_gather_into_tensor(gathered.view(world * m, ns), out)

    comm_stream = torch.cuda.Stream()

    def pipelined_step(i):
        wq, ws, _ = wsets[i]
        parallel.column_parallel_linear_pipelined(a4, asf, ag, wq, ws, wg, gathered, chunks=4,
                                                  comm_stream=comm_stream)

    def barrier():
        dist.barrier()

    # GEMM alone (graph), then GEMM + all-gather (eager: NCCL collectives are enqueued directly)
    secs_gemm, _, _ = time_graph(gemm_only, n_sets, args.steps, args.warmup, barrier)
    for i in range(max(args.warmup, 3)):
        full_step(i % n_sets)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            full_step(i % n_sets)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    secs_serial = e0.elapsed_time(e1) * 1e-3
    # same work with the exchange overlapped: 4 row blocks, sends of block i under the GEMM of block i+1
    for i in range(max(args.warmup, 3)):
        pipelined_step(i % n_sets)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clk:
        t0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            pipelined_step(i % n_sets)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    secs_pipe = e0.elapsed_time(e1) * 1e-3
    # the same step with the all-gather fused into the GEMM epilogue: every tile is stored into every
    # rank's [M, N] buffer over NVLink, a one-element all-reduce closes the step
    peer = parallel.PeerOutput(m, n, torch.bfloat16)
    sync = torch.zeros(1, dtype=torch.float32, device="cuda")

    last = {}

    def fused_step(i):
        wq, ws, _ = wsets[i]
        last["out"] = parallel.column_parallel_linear_fused(a4, asf, ag, wq, ws, wg, peer, sync=sync)

    for t_ in peer.tensors:
        t_.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    for i in range(max(args.warmup, 3)):
        fused_step(i % n_sets)
    torch.cuda.synchronize()
    full_step(0)
    torch.cuda.synchronize()
    fused_ok = all(torch.equal(last["out"][:, r * ns:(r + 1) * ns], gathered[r]) for r in range(world))
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clk:
        t0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            fused_step(i % n_sets)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    secs = e0.elapsed_time(e1) * 1e-3
    # NVLink ceiling measured in this run: every rank copies 256 MiB from its own memory into the next rank's
    # output buffer (the peer mapping the fused epilogue stores through; cudaMemcpyAsync device-to-device), all
    # ranks at once, so every GPU sends on its links while it receives; CUDA events, 5 repetitions
    ring_bytes = 256 << 20
    ring_src = torch.empty(ring_bytes, dtype=torch.uint8, device="cuda")
    holder = type("_Mem", (), {})()
    holder.__cuda_array_interface__ = {"shape": (ring_bytes,), "typestr": "|u1", "version": 3, "strides": None,
                                       "data": (peer.ptrs[(rank + 1) % world], False)}
    ring_dst = torch.as_tensor(holder, device=torch.device("cuda", local))

    def ring():
        ring_dst.copy_(ring_src, non_blocking=True)

    for _ in range(2):
        ring()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(5):
        ring()
    e1.record()
    torch.cuda.synchronize()
    secs_ring = e0.elapsed_time(e1) * 1e-3 / 5
    dist.barrier()
    del ring_dst, holder, ring_src
    t = torch.tensor([secs, secs_gemm, secs_serial, secs_pipe, 0.0 if fused_ok else 1.0, secs_ring], dtype=torch.float64,
                     device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs, secs_gemm, secs_serial, secs_pipe, fused_bad, secs_ring = (float(v) for v in t)
    peer.close()
    dist.barrier()
    if rank == 0:
        value = flops / (secs / args.steps) / 1e12
        gemm_tflops = flops / (secs_gemm / args.steps) / 1e12
        recv_bytes = (world - 1) * m * ns * 2
        gather_s = max(secs_serial - secs_gemm, 1e-9) / args.steps
        fp4_proxy_peak = 4.0 * peaks["bf16_tflops"] * world
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": c5_workload(world),
                       "l2": f"{n_sets} weight/output sets rotated per rank",
                       "timing": "CUDA events on each rank, max over ranks"},
            "gemm_only_tflops": gemm_tflops,
            "serial_gemm_then_all_gather_tflops": flops / (secs_serial / args.steps) / 1e12,
            "pipelined_send_recv_tflops": flops / (secs_pipe / args.steps) / 1e12,
            "exchange": "all-gather fused into the GEMM epilogue: each tile is staged in shared memory once and stored "
                        "to every rank's [M, N] buffer with TMA stores (the peers' over NVLink), closed by a "
                        "one-element all-reduce; the serial NCCL all-gather and a 4-block send/recv pipeline are "
                        "timed beside it",
            "fused_output_equals_nccl_all_gather": fused_bad == 0.0,
            "nvlink": {"sent_bytes_per_gpu": recv_bytes, "gbs_per_gpu_per_direction": recv_bytes / (secs / args.steps) / 1e9,
                       "measured_peer_copy_gbs_per_direction": (256 << 20) / secs_ring / 1e9,
                       "frac_of_measured_peer_copy": recv_bytes / (secs / args.steps) / ((256 << 20) / secs_ring),
                       "floor_ms_at_measured_peer_copy": recv_bytes / ((256 << 20) / secs_ring) * 1e3,
                       "note": "the output is replicated on every rank, so each GPU sends and receives "
                               "(w-1)/w x M x N x 2 bytes per step whatever the GEMM does"},
            "gemm_only_per_gpu_frac_of_nominal_fp4": gemm_tflops / world / NOMINAL_FP4_TFLOPS,
            "all_gather": {"recv_bytes_per_gpu": recv_bytes, "exposed_ms": gather_s * 1e3,
                           "recv_gbs_per_gpu": recv_bytes / gather_s / 1e9},
            "roofline": {"bound": "tensor", "achieved": gemm_tflops, "peak": fp4_proxy_peak, "unit": "TFLOP/s",
                         "frac": gemm_tflops / fp4_proxy_peak, "traffic": None,
                         "traffic_note": "DRAM bytes need ncu, which never wraps a multi-rank run; NVLink bytes per GPU and "
                                         "step are algorithmic, see nvlink.sent_bytes_per_gpu",
                         "peak_note": f"{world} x 4 x {peaks['source']} bf16 burst; GEMM-only"},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "activations and weights are layer-resident in this variant; see the 1-GPU line for host copies"},
            "clocks": clk.summary(t0, t1),
            "gpu_launches": args.steps,
        }
        print(json.dumps(line))
    dist.destroy_process_group()


def run_profile_case(case):
    """One small workload, three launches, no timing: the command line that ncu wraps."""
    from ac4k_kernel_b200 import _cuda_ops, _lib, ops
    from ac4k_kernel_b200.ops.quant import _global_scale
    torch.cuda.set_device(0)
    if case.startswith("gemm"):
        dims = {"gemm-c2": (4096, 4096, 4096), "gemm-8k": (8192, 8192, 8192), "gemm-decode": (16, 8192, 8192)}[case]
        m, n, k = dims
        a = activations((m, k), 0, 0.005, 30.0, "cuda")
        w = weights((n, k), 1, "cuda")
        a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
        w4, wsf, wg = ops.quantize(w, 0, 1, sf_layout="128x4")
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        for _ in range(3):
            _cuda_ops.linear_nvfp4(out, a4, asf, ag, w4, wsf, wg, None)
    elif case == "rope3d":
        f, h, w = 21, 45, 80
        x = torch.randn((1, f * h * w, 40, 128), dtype=torch.bfloat16, device="cuda",
                        generator=torch.Generator(device="cuda").manual_seed(9567))
        grid = torch.tensor([[f, h, w]], dtype=torch.int32, device="cuda")
        ang = torch.outer(torch.arange(1024, dtype=torch.float64),
                          1.0 / torch.pow(torch.tensor(10000.0, dtype=torch.float64), torch.arange(0, 128, 2, dtype=torch.float64) / 128))
        freqs = torch.polar(torch.ones_like(ang), ang).cuda()
        out = torch.empty_like(x)
        for _ in range(3):
            ops.rope3d(x, grid, freqs, out)
    elif case in ("mha-int8", "quant-attn"):
        import math
        from ac4k_kernel_b200.ops.attention import _int8_quantize
        g = torch.Generator(device="cuda").manual_seed(9567)
        n, h = (8192, 16) if case == "mha-int8" else (75600, 40)
        q, k, v = (torch.randn((1, n, h, 128), dtype=torch.bfloat16, device="cuda", generator=g) for _ in range(3))
        for _ in range(3):
            q8, q8s = _int8_quantize(q, "BNHD", 1, BLOCK_SIZE=64)
            k8, k8s = _int8_quantize(k, "BNHD", 1, BLOCK_SIZE=128)
            v8, v8s = ops.quantize(v, 3, 1, swizzle=True, max_scale=2.25, precision="fp8e4m3")
        if case == "mha-int8":
            out = torch.empty_like(q)
            for _ in range(3):
                _cuda_ops.mha_int8_x_fp8_fwd(out.permute(0, 2, 1, 3), q8, q8s, 64, k8, k8s, 128, v8, v8s, 1 / math.sqrt(128))
    elif case == "mha":
        import math
        g = torch.Generator(device="cuda").manual_seed(9567)
        q, k, v = (torch.randn((1, 8192, 16, 128), dtype=torch.bfloat16, device="cuda", generator=g) for _ in range(3))
        qq, qs, qg = ops.quantize(q, 1, 3, sf_layout="128x4")
        kq, ks, kg = ops.quantize(k, 1, 3, sf_layout="128x4")
        vq, vs, vg = ops.quantize(v, 3, 1, swizzle=True, sf_layout="128x4")
        out = torch.empty_like(q)
        for _ in range(3):
            _cuda_ops.mha_nvfp4_fwd(out.permute(0, 2, 1, 3), qq, qs, qg, kq, ks, kg, vq, vs, vg, 1 / math.sqrt(128))
    else:
        m, k = 32768, 8192
        x = activations((m, k), 0, 0.01, 50.0, "cuda")
        for _ in range(3):
            if case == "quant-c4":
                ops.quantize(x, 0, 1, sf_layout="128x4")
            elif case == "quant-c4-fp8":
                ops.quantize(x, 0, 1, precision="fp8e4m3")
            else:
                ops.quantize(x, 0, 1, precision="int8")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": case, "device_status": _lib.device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-case", default=None,
                    choices=["gemm-c2", "gemm-8k", "gemm-decode", "mha", "mha-int8", "quant-attn", "rope3d", "quant-c4", "quant-c4-fp8", "quant-c4-int8"],
                    help="run one small workload three times and exit (for ncu)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback "
                         "(use --impl reference for the CPU emulation)")
    peaks = load_peaks()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        run_multi(args, peaks)
    else:
        run_single(args, peaks)


if __name__ == "__main__":
    main()
