#!/usr/bin/env python
"""Benchmark of the quantised-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input: the MXFP8 A8W8 GEMM
out[M,N] = A[M,K] . B[N,K]^T with UE8M0 scales per 1x32 along K, N = K = 4096, M = 8192, bf16 output
(the largest point of the reference's MXFP8 configuration).  Inputs come from bf16 N(0,1) data,
seeded, quantised with scale = 2^ceil(log2(amax/448)).  `value` is whole-job TFLOP/s with inputs
resident in HBM; `e2e` is the same metric through the operator call with pinned HOST buffers for the
step's activations, their scales and the output (the weight, a model parameter, stays resident).
With N > 1 every rank owns one 4096-column shard of a weight N times as wide (no collective on the
data path): weak scaling.  `sweep` adds the per-M figures of the other configurations.

`--impl reference` times the reference's CPU path (dequantise to fp32 -> matmul -> bf16; the torch-on-CPU
restatement under oracle/) on the host cores, on a bounded row slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_DIM, K_DIM, M_DIM = 4096, 4096, 8192
METRIC = "GEMM TFLOPS/GPU (MXFP8 A8W8, N=K=4096, M=8192)"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload's kernel, from the ncu capture
# summarised under profiles/ (52.0 MB read + 32.0 MB written; the 126 MB L2 holds part of the 119 MB working set)
NCU_TRAFFIC_BYTES = 84.0e6
NOMINAL = {"bf16": 2250.0, "mxfp8": 4500.0, "mxfp4": 9000.0, "a8w4": 4500.0, "hbm_gbs": 8000.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------- inputs
def quantised_problem(torch, ab, M, N, K, seed, device, kind="mxfp8"):
    """Seeded bf16 N(0,1) data quantised by the library's (oracle-exact) torch quantisers on the GPU,
    then put in the wire layouts the operators take."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(M, K, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    if kind == "mxfp8":
        xq, xs = ab.per_1x32_f8_scale_f8_quant(x, scale_type=ab.dtypes.fp8_e8m0)
        wq, ws = ab.per_1x32_f8_scale_f8_quant(w, scale_type=ab.dtypes.fp8_e8m0)
        return (xq, ab.shuffle_mxfp8fp4_b(wq), ab.shuffle_mxfp8fp4_scale(xs.view(torch.uint8)),
                ab.shuffle_mxfp8fp4_scale(ws.view(torch.uint8)))
    if kind == "mxfp4":
        xq, xs = ab.per_1x32_f4_quant(x, shuffle=True)
        wq, ws = ab.per_1x32_f4_quant(w, shuffle=True)
        return (xq, ab.shuffle_weight(wq, layout=(16, 16)), xs, ws)
    raise ValueError(kind)


def algorithmic_bytes(kind, M, N, K):
    if kind == "bf16":
        return 2 * (M * K + N * K + M * N)
    if kind == "mxfp8":
        return M * K + N * K + (M + N) * K // 32 + 2 * M * N
    if kind == "mxfp4":
        return (M * K + N * K) // 2 + (M + N) * K // 32 + 2 * M * N
    return M * K + N * K // 2 + (M + N) * K // 32 + 2 * M * N


def time_calls(torch, fn, arg_sets, iters, warmup):
    """Device time per call in microseconds: CUDA events on the launching (current) stream, rotating
    argument sets larger than L2 between iterations."""
    n = len(arg_sets)
    for i in range(warmup):
        fn(*arg_sets[i % n])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(*arg_sets[i % n])
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def graph_time_calls(torch, fn, arg_sets, iters, warmup):
    """Same, but the calls are replayed from one CUDA graph so that host launch cost does not hide
    the device time of microsecond-sized kernels."""
    n = len(arg_sets)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        # warm up on the capture stream itself: the split-K workspace is per stream and may not grow
        # while the stream is being captured
        for i in range(max(warmup, n)):
            fn(*arg_sets[i % n])
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                fn(*arg_sets[i % n])
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def kernel_in_use(ab, kind, M, N, K):
    """Name of the kernel configuration the operator picks: the tuned table's row, else the heuristic."""
    from aiter_b200 import gemm_op_a4w4, gemm_op_a8w4, gemm_op_a8w8

    row = None
    if kind == "mxfp8":
        row = gemm_op_a8w8._mxfp8_table.lookup(M, N, K)
    elif kind == "mxfp4":
        row = gemm_op_a4w4.get_GEMM_config(M, N, K)
    elif kind == "a8w4":
        row = gemm_op_a8w4.get_A8W4_config(M, N, K)
    if row is not None and row.get("kernelName"):
        name = str(row["kernelName"])
        split = row.get("splitK")
        return name if "_k" in name or not split else f"{name}_k{int(split)}"
    return ab.heuristic_name({"bf16": 0, "mxfp8": 1, "mxfp4": 2, "a8w4": 3}[kind], M, N, K)[0]


def rotating_sets(make, bytes_per_set, l2_bytes=126e6):
    n = max(2, min(24, int(2.2 * l2_bytes // max(bytes_per_set, 1)) + 1))
    return [make(i) for i in range(n)]


# --------------------------------------------------------------------------------------- sweep
def run_case(torch, ab, device, spec, steps, warmup):
    """Profiling aid: one sweep case, `kind:M:N:K` with kind in mxfp8 / mxfp4 / a8w4 / bf16 / blockscale_fp32 /
    blockscale_e8m0 / quant_mxfp4 / quant_mxfp8 (N ignored for the quantiser), launched `steps` times on the current stream; prints one JSON line."""
    kind, M, N, K = spec.split(":")
    M, N, K = int(M), int(N), int(K)

    def rand_u8(lo, hi, *shape):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=device)

    if kind == "mxfp8":
        args = (rand_u8(0, 0x78, M, K).view(torch.float8_e4m3fn), rand_u8(0, 0x78, N, K).view(torch.float8_e4m3fn),
                rand_u8(120, 130, (M + 31) // 32 * 32, K // 32), rand_u8(120, 130, N, K // 32))
        fn = lambda a, b, sa, sb: ab.gemm_a8w8_mxfp8(a, b, sa, sb, a_preshuffle=False)  # noqa: E731
    elif kind == "mxfp4":
        kb = (K // 32 + 7) // 8 * 8
        args = (rand_u8(0, 256, M, K // 2), rand_u8(0, 256, N, K // 2), rand_u8(120, 130, (M + 255) // 256 * 256, kb),
                rand_u8(120, 130, (N + 255) // 256 * 256, kb))
        fn = lambda a, b, sa, sb: ab.gemm_a4w4(a, b, sa, sb)  # noqa: E731
    elif kind == "a8w4":
        args = (rand_u8(0, 0x78, M, K).view(torch.float8_e4m3fn), rand_u8(0, 256, N, K // 2),
                rand_u8(120, 130, (M + 31) // 32 * 32, K // 32), rand_u8(120, 130, N, K // 32))
        fn = lambda a, b, sa, sb: ab.gemm_a8w4_mxfp8(a, b, sa, sb, a_preshuffle=False)  # noqa: E731
    elif kind == "bf16":
        args = (torch.randn(M, K, device=device).to(torch.bfloat16) * 0.1, torch.randn(N, K, device=device).to(torch.bfloat16) * 0.1)
        fn = lambda a, b: ab.tgemm.mm(a, b)  # noqa: E731
    elif kind in ("quant_mxfp4", "quant_mxfp8"):
        args = (torch.randn(M, K, device=device).to(torch.bfloat16),)
        kw = dict(quant_dtype=ab.dtypes.fp4x2, shuffle=True) if kind == "quant_mxfp4" else dict(
            quant_dtype=ab.dtypes.fp8, scale_type=ab.dtypes.fp8_e8m0, shuffle=2)
        fn = lambda x: ab.per_1x32_mx_quant_hip(x, **kw)  # noqa: E731
    elif kind in ("blockscale_fp32", "blockscale_e8m0"):
        kb, nb = K // 128, (N + 127) // 128
        scales = (torch.rand(M, kb, device=device) + 0.5, torch.rand(nb, kb, device=device) + 0.5) if kind.endswith("fp32") else (
            rand_u8(124, 130, M, kb).view(ab.dtypes.fp8_e8m0), rand_u8(124, 130, nb, kb).view(ab.dtypes.fp8_e8m0))
        args = (rand_u8(0, 0x78, M, K).view(torch.float8_e4m3fn), rand_u8(0, 0x78, N, K).view(torch.float8_e4m3fn), *scales)
        fn = lambda a, b, xs, ws: ab.gemm_a8w8_blockscale(a, b, xs, ws)  # noqa: E731
    else:
        raise SystemExit(f"unknown case kind {kind}")
    us = time_calls(torch, fn, [args], steps, warmup)
    if kind.startswith("quant"):
        kernel = "quant_mx_kernel"
    elif kind.startswith("blockscale"):
        kernel = "gemm_a8w8_blockscale" + ("_fewrows_kernel" if M <= 64 else " -> mxfp8" if kind.endswith("e8m0")
                                           else "_pair_kernel" if M > 128 else "_kernel")
    else:
        kernel = kernel_in_use(ab, kind, M, N, K)
    print(json.dumps({"case": spec, "us_per_call": round(us, 2), "steps": steps, "warmup": warmup, "kernel": kernel}))


def run_sweep(torch, ab, device, peaks):
    """Per-M device time of the other benchmark configurations (graph-replayed, rotating buffers).
    The cases run in ascending order of work after a second of idle time, and are reported in the order they are
    declared: right after a long tensor-bound case the GPU sits at its power cap (SM clock ~1.45 GHz instead of
    1.97 GHz for some milliseconds), which would inflate the microsecond-sized decode cases by 10-30 %."""
    import time

    jobs = []  # (work, thunk returning the row)

    def rand_u8(lo, hi, *shape):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=device)

    def add(kind, M, N, K, fn, make):
        def job():
            b = algorithmic_bytes(kind, M, N, K)
            sets = rotating_sets(make, b)
            us = graph_time_calls(torch, fn, sets, 20, 3)
            tf = 2.0 * M * N * K / us / 1e6
            gbs = b / us / 1e3
            peak_tf = peaks["bf16"] * {"bf16": 1, "mxfp8": 2, "a8w4": 2, "mxfp4": 4}[kind]
            return {"kind": kind, "M": M, "N": N, "K": K, "us": round(us, 2), "tflops": round(tf, 1), "gbs": round(gbs, 1),
                    "frac_tensor": round(tf / peak_tf, 4), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
                    "kernel": kernel_in_use(ab, kind, M, N, K)}

        jobs.append((2.0 * M * N * K, job))

    # bf16 a16w16 (the reference's CPU-runnable case)
    add("bf16", 64, 1024, 1024, lambda a, b: ab.tgemm.mm(a, b),
        lambda i: (torch.randn(64, 1024, device=device).to(torch.bfloat16) * 0.1, torch.randn(1024, 1024, device=device).to(torch.bfloat16) * 0.1))
    # MXFP8, N = K = 4096
    for M in (1, 16, 128, 1024, 8192):
        add("mxfp8", M, 4096, 4096, lambda a, b, sa, sb: ab.gemm_a8w8_mxfp8(a, b, sa, sb, a_preshuffle=False),
            lambda i, M=M: (rand_u8(0, 0x78, M, 4096).view(torch.float8_e4m3fn), rand_u8(0, 0x78, 4096, 4096).view(torch.float8_e4m3fn),
                            rand_u8(120, 130, (M + 31) // 32 * 32, 128), rand_u8(120, 130, 4096, 128)))
    # MXFP4, DeepSeek-V3-like (N, K)
    for (N, K) in ((7168, 2048), (24576, 1536), (7168, 16384)):
        for M in (1, 32, 256, 4096, 16384):
            kb = (K // 32 + 7) // 8 * 8
            add("mxfp4", M, N, K, lambda a, b, sa, sb: ab.gemm_a4w4(a, b, sa, sb),
                lambda i, M=M, N=N, K=K, kb=kb: (rand_u8(0, 256, M, K // 2), rand_u8(0, 256, N, K // 2),
                                                 rand_u8(120, 130, (M + 255) // 256 * 256, kb), rand_u8(120, 130, (N + 255) // 256 * 256, kb)))
    # MXFP8 activations x MXFP4 weights, N = K = 8192
    for M in (1, 16, 128, 1024, 4096, 16384):
        add("a8w4", M, 8192, 8192, lambda a, b, sa, sb: ab.gemm_a8w4_mxfp8(a, b, sa, sb, a_preshuffle=False),
            lambda i, M=M: (rand_u8(0, 0x78, M, 8192).view(torch.float8_e4m3fn), rand_u8(0, 256, 8192, 4096),
                            rand_u8(120, 130, (M + 31) // 32 * 32, 256), rand_u8(120, 130, 8192, 256)))
    # FP8 with 128-block scales, N = K = 4096: fp32 scales (promotion kernel) and e8m0 scales (MXFP8 kernel)
    for M in (16, 1024, 8192):
        for tag, mk in (("blockscale_fp32", lambda M: (torch.rand(M, 32, device=device) + 0.5, torch.rand(32, 32, device=device) + 0.5)),
                        ("blockscale_e8m0", lambda M: (rand_u8(124, 130, M, 32).view(ab.dtypes.fp8_e8m0), rand_u8(124, 130, 32, 32).view(ab.dtypes.fp8_e8m0)))):
            def job(M=M, tag=tag, mk=mk):
                sets = rotating_sets(lambda i: (rand_u8(0, 0x78, M, 4096).view(torch.float8_e4m3fn),
                                                rand_u8(0, 0x78, 4096, 4096).view(torch.float8_e4m3fn), *mk(M)),
                                     algorithmic_bytes("mxfp8", M, 4096, 4096))
                us = graph_time_calls(torch, lambda a, b, xs, ws: ab.gemm_a8w8_blockscale(a, b, xs, ws), sets, 20, 3)
                tf = 2.0 * M * 4096 * 4096 / us / 1e6
                return {"kind": tag, "M": M, "N": 4096, "K": 4096, "us": round(us, 2), "tflops": round(tf, 1),
                        "gbs": round(algorithmic_bytes("mxfp8", M, 4096, 4096) / us / 1e3, 1), "frac_tensor": round(tf / (2 * peaks["bf16"]), 4),
                        "frac_hbm": round(algorithmic_bytes("mxfp8", M, 4096, 4096) / us / 1e3 / peaks["hbm_gbs"], 4),
                        "kernel": "gemm_a8w8_blockscale" + ("_fewrows_kernel" if M <= 64 else "_pair_kernel" if tag.endswith("fp32") and M > 128
                                                            else "_kernel" if tag.endswith("fp32") else " -> mxfp8")}

            jobs.append((2.0 * M * 4096 * 4096, job))
    # fused activation quantiser (bf16 -> MX data + scales in the GEMM's layout): HBM-bound
    for (kind, M, K, kw) in (("quant_mxfp4", 16384, 16384, dict(quant_dtype=ab.dtypes.fp4x2, shuffle=True)),
                             ("quant_mxfp8", 8192, 4096, dict(quant_dtype=ab.dtypes.fp8, scale_type=ab.dtypes.fp8_e8m0, shuffle=2)),
                             ("quant_mxfp4", 32, 16384, dict(quant_dtype=ab.dtypes.fp4x2, shuffle=True))):
        def job(kind=kind, M=M, K=K, kw=kw):
            b = int(M * K * 2 + M * K * (0.5 if kind == "quant_mxfp4" else 1.0) + M * K / 32)
            sets = rotating_sets(lambda i: (torch.randn(M, K, device=device).to(torch.bfloat16),), M * K * 2)
            us = graph_time_calls(torch, lambda x: ab.per_1x32_mx_quant_hip(x, **kw), sets, 20, 3)
            return {"kind": kind, "M": M, "N": 0, "K": K, "us": round(us, 2), "tflops": 0.0, "gbs": round(b / us / 1e3, 1),
                    "frac_tensor": 0.0, "frac_hbm": round(b / us / 1e3 / peaks["hbm_gbs"], 4), "kernel": "quant_mx_kernel"}

        jobs.append((float(M) * K, job))  # memory-bound: sorts among the small cases
    torch.cuda.synchronize()
    time.sleep(1.0)
    rows = [None] * len(jobs)
    for idx in sorted(range(len(jobs)), key=lambda i: jobs[i][0]):
        rows[idx] = jobs[idx][1]()
    return rows


# --------------------------------------------------------------------------------------- CPU path
def cpu_reference_step(sample_rows, seed=0):
    """Builds a bounded sample (the first `sample_rows` rows of the workload) and returns a callable
    running the reference's CPU algorithm (torch ops on every host thread) on it plus its flops."""
    import torch

    from oracle import torch_ref as tr
    from oracle import mx_oracle as ox

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(sample_rows, K_DIM, generator=g).to(torch.bfloat16).float().numpy()
    w = torch.randn(N_DIM, K_DIM, generator=g).to(torch.bfloat16).float().numpy()
    xq, xs = (torch.from_numpy(t) for t in ox.quant_mxfp8(x))
    wq, ws = (torch.from_numpy(t) for t in ox.quant_mxfp8(w))
    return (lambda: tr.gemm_a8w8_mxfp8(xq, wq, xs, ws)), 2.0 * sample_rows * N_DIM * K_DIM


def time_cpu(sample_rows, repeats):
    step, flops = cpu_reference_step(sample_rows)
    step()
    t0 = time.perf_counter()
    for _ in range(repeats):
        step()
    dt = (time.perf_counter() - t0) / repeats
    return flops / dt / 1e12, dt


def run_reference(args, rank, world):
    if rank != 0:
        return
    import torch

    cores = torch.get_num_threads()
    sample_rows = 256
    for _ in range(max(args.warmup, 1) - 1):
        time_cpu(sample_rows, 1)
    tf, dt = time_cpu(sample_rows, max(args.steps, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3 x e4m3 -> f32 (dequantised fp32 matmul on the CPU)", "data": "synthetic",
        "config": {"workload": f"mxfp8_a8w8 M={M_DIM} N={N_DIM} K={K_DIM} (CPU sample: first {sample_rows} rows of M)"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_rows} of {M_DIM} rows of M, full N and K; dequantise + fp32 matmul + bf16 cast"},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------- ours
def run_ours(args, rank, world, local_rank):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GEMM path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import aiter_b200 as ab

    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    if args.case:
        run_case(torch, ab, device, args.case, args.steps, args.warmup)
        return
    peaks = measured_peaks()
    M, N, K = M_DIM, N_DIM, K_DIM
    flops = 2.0 * M * N * K
    bytes_alg = algorithmic_bytes("mxfp8", M, N, K)

    # rotating input sets, each rank its own weight shard (seeded by rank)
    def make(i):
        a, b, sa, sb = quantised_problem(torch, ab, M, N, K, seed=1000 * rank + i, device=device)
        return (a, b, sa, sb)

    sets = rotating_sets(make, bytes_alg)
    fn = lambda a, b, sa, sb: ab.gemm_a8w8_mxfp8(a, b, sa, sb, a_preshuffle=False)  # noqa: E731

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        fn(*sets[i % len(sets)])
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = ab.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        fn(*sets[i % len(sets)])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = ab.launch_count() - launches0
    clocks = sampler.stop() if sampler is not None else None
    status = ab.device_status(local_rank)

    # ---- end to end: pinned host activations -> device, GEMM, output -> pinned host, every step.  The three legs of
    # consecutive steps overlap (copy-in stream, compute stream, copy-out stream, two buffer sets): the figure is the
    # sustained rate of the whole pipeline, bounded by the slowest leg (the 67 MB result crossing PCIe).
    a0, b0, sa0, sb0 = sets[0]
    n_buf = 2
    h_a = [torch.empty(a0.shape, dtype=torch.uint8).pin_memory() for _ in range(n_buf)]
    h_sa = [torch.empty(sa0.shape, dtype=torch.uint8).pin_memory() for _ in range(n_buf)]
    h_out = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(n_buf)]
    for i in range(n_buf):
        h_a[i].copy_(a0.view(torch.uint8).cpu())
        h_sa[i].copy_(sa0.cpu())
    d_a = [torch.empty_like(a0) for _ in range(n_buf)]
    d_sa = [torch.empty_like(sa0) for _ in range(n_buf)]
    d_out = [None] * n_buf
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]        # inputs of buffer b are on the device
    ev_gemm = [torch.cuda.Event() for _ in range(n_buf)]      # the GEMM on buffer b is done (inputs free, output ready)
    ev_out = [torch.cuda.Event() for _ in range(n_buf)]       # the result of buffer b is in host memory
    for b in range(n_buf):
        ev_gemm[b].record(s_main)
        ev_out[b].record(s_out)

    def e2e_step(i):
        b = i % n_buf
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_gemm[b])  # the previous GEMM on this buffer has read its inputs
            d_a[b].view(torch.uint8).copy_(h_a[b], non_blocking=True)
            d_sa[b].copy_(h_sa[b], non_blocking=True)
            ev_in[b].record(s_in)
        s_main.wait_event(ev_in[b])
        s_main.wait_event(ev_out[b])     # the previous result held by this slot has left the device
        d_out[b] = ab.gemm_a8w8_mxfp8(d_a[b], b0, d_sa[b], sb0, a_preshuffle=False)
        ev_gemm[b].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_gemm[b])
            # d_out[b] stays referenced until this slot's next GEMM, which first waits for ev_out[b] on the compute
            # stream: the allocator can hand the block back to that stream safely without record_stream
            h_out[b].copy_(d_out[b], non_blocking=True)
            ev_out[b].record(s_out)

    e2e_steps = 0 if args.kernel_only else max(6, min(args.steps, 20))
    for i in range(min(4, e2e_steps)):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = max(time.perf_counter() - t0, 1e-9)
    h_a, h_sa, h_out = h_a[0], h_sa[0], h_out[0]
    h2d, d2h = h_a.numel() + h_sa.numel(), h_out.numel() * 2

    # max over ranks
    if dist is not None:
        t = torch.tensor([ms, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    tflops = flops * args.steps * world / (ms * 1e-3) / 1e12
    e2e_tflops = flops * e2e_steps * world / e2e_s / 1e12

    sweep, cpu = None, None
    if rank == 0:
        per_launch_us = ms * 1e3 / args.steps
        kernel_tf = flops / per_launch_us / 1e6
        peak_fp8 = 2.0 * peaks["bf16"]
        roofline = {
            "bound": "tensor", "achieved": round(kernel_tf, 1), "peak": round(peak_fp8, 1), "unit": "TFLOP/s",
            "frac": round(kernel_tf / peak_fp8, 4), "traffic": NCU_TRAFFIC_BYTES, "traffic_unit": "bytes per launch",
            "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16']} TFLOP/s); FP8 tensor rate is twice the bf16 rate",
            "frac_of_nominal_4500": round(kernel_tf / NOMINAL["mxfp8"], 4),
            "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": bytes_alg,
            "avg_launch_us": round(per_launch_us, 2),
        }
        if not (args.no_sweep or args.kernel_only):
            sweep = run_sweep(torch, ab, device, peaks)
        if world == 1 and not args.kernel_only:  # the CPU baseline is a single-GPU-run figure
            cpu_tf, cpu_dt = time_cpu(256, 3)
            cpu = {"value": round(cpu_tf, 4), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"256 of {M} rows of M, full N and K ({cpu_dt * 1e3:.0f} ms per pass, torch-on-CPU restatement of the reference path)"}
        line = {
            "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 x e4m3 (UE8M0 scales) -> f32 accumulate -> bf16", "data": "synthetic",
            "config": {"workload": f"mxfp8_a8w8 M={M} N={N} K={K} per GPU (N-sharded weight, one 4096-column shard per rank)",
                       "l2_policy": f"{len(sets)} rotating input sets of {bytes_alg / 1e6:.0f} MB (> 126 MB L2 in total)",
                       "kernel": kernel_in_use(ab, "mxfp8", M, N, K), "e2e_copies": "activations + their scales H2D, output D2H, weight resident; the three legs of consecutive steps overlap on three streams"},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "clocks": clocks, "device_status": list(status),
        }
        if sweep is not None:
            line["sweep"] = sweep
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-M table of the other configurations")
    ap.add_argument("--kernel-only", action="store_true",
                    help="profiling aid: only the device-timed GEMM loop (no end-to-end leg, sweep or CPU baseline)")
    ap.add_argument("--case", default="", help="profiling aid: run one sweep case only, kind:M:N:K (see run_case)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
