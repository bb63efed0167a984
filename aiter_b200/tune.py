"""Tuner: measures every candidate kernel configuration for a list of (M, N, K) shapes on the GPU it runs on
and writes the winners into a tuned table in the reference's CSV schema.

    python -m aiter_b200.tune --family a8w8_mxfp8 --baseline            # the benchmark shapes
    python -m aiter_b200.tune --family a4w4 --shapes "32,7168,2048;4096,7168,2048" -o my.csv
    python -m aiter_b200.tune --family bf16 -i aiter_b200/configs/bf16_untuned_gemm.csv          # shapes tgemm recorded
    python -m aiter_b200.tune --family a4w4 --run_config my.csv         # time the production operator with a table, no tuning
    python -m aiter_b200.tune --family a4w4 --baseline --compare --update_improved --min_improvement_pct 3
    python -m aiter_b200.tune --family a4w4 --baseline --mp 8 --timeout 600   # shapes spread over 8 GPUs, one worker each

Same flow as the reference's tuners (aiter/utility/base_tuner.py:1537-1722,
csrc/ck_gemm_a4w4_blockscale/gemm_a4w4_blockscale_tune.py): candidates come from the kernel menu, every
candidate is checked against a torch reference before it may win (errRatio gate, tolerance rtol = atol = 1e-2),
timing is device time with rotating inputs larger than L2 (CUDA-graph replay), rows carry
us / tflops / bw / errRatio, shapes already present in the output file are skipped unless --retune, and the
file is rewritten after every shape so an interrupted run can be resumed.  --run_config, --compare / --update_improved
/ --min_improvement_pct and the shape file (-i) follow aiter/utility/base_tuner.py:208-240,571-583; --mp runs one worker
process per GPU with a per-worker watchdog and gives the shapes of a worker that died or ran out of time to another one
once, as aiter/utility/mp_tuner.py:168-189 restarts its pool.
"""
from __future__ import annotations

import argparse
import csv
import os
import subprocess
import sys
import tempfile
import time

import torch

from . import _ffi, config, dtypes, fp4_utils, shuffle

FAMILIES = {
    # family -> (table name, problem kind id of aiter_b200_heuristic_name, csv header)
    "a4w4": ("a4w4", 2),
    "a8w8_mxfp8": ("a8w8_mxfp8", 1),
    "a8w4_mxfp8": ("a8w4_mxfp8", 3),
    "bf16": ("bf16", 0),
    "a8w8_blockscale": ("a8w8_blockscale", 1),
    "a8w8_blockscale_bpreshuffle": ("a8w8_blockscale_bpreshuffle", 1),
}
BLOCKSCALE_HEADER = ["gfx", "cu_num", "M", "N", "K", "libtype", "kernelId", "splitK", "us", "kernelName", "tflops", "bw", "errRatio"]
BLOCKSCALE_VARIANTS = {"bs_fewrows": 1, "bs_128x128": 2, "bs_256x256": 3, "bs_256x128": 4}
HEADER = ["gfx", "cu_num", "M", "N", "K", "kernelId", "splitK", "us", "kernelName", "tflops", "bw", "errRatio"]
BF16_HEADER = ["gfx", "cu_num", "M", "N", "K", "bias", "dtype", "outdtype", "scaleAB", "bpreshuffle", "libtype", "solidx", "splitK",
               "us", "kernelName", "err_ratio", "tflops", "bw"]
BASELINE_SHAPES = {
    "bf16": [(64, 1024, 1024), (1024, 8192, 8192), (8192, 8192, 8192)],
    "a8w8_mxfp8": [(m, 4096, 4096) for m in (1, 16, 128, 1024, 8192)],
    "a4w4": [(m, n, k) for (n, k) in ((7168, 2048), (24576, 1536), (7168, 16384)) for m in (1, 32, 256, 4096, 16384)] + [(16384, 7168, 7168)],
    "a8w4_mxfp8": [(1 << e, 8192, 8192) for e in range(15)],
    "a8w8_blockscale": [(m, 4096, 4096) for m in (1, 16, 128, 1024, 8192)],
    "a8w8_blockscale_bpreshuffle": [(m, 4096, 4096) for m in (1, 16, 128, 1024, 8192)],
}
BN_MENU = [16, 32, 64, 128, 256, 192, 224, 96, 160]


def kernel_id(pair: int, swap: int, bn: int, stages: int) -> int:
    return pair * 1000 + swap * 100 + BN_MENU.index(bn) * 10 + stages


def kernel_name(pair: int, swap: int, bn: int, stages: int, log2_splitk: int | None = None) -> str:
    name = f"tc5_{256 if pair else 128}x{bn}_{'t' if swap else 'n'}_s{stages}"
    return name if log2_splitk is None else f"{name}_k{log2_splitk}"


def blockscale_candidates(M: int, N: int, K: int):
    """Kernel names of the fp32-scale kernels worth timing: which kernel and its K split ("" = the launcher's own model)."""
    kb = K // 128
    names = [""]
    if M <= 256 or (M <= 1024 and N <= 1024):  # (beyond 64 rows: several tiles of 64 rows on the same weight tile)
        names += [f"bs_fewrows_k{s}" for s in range(0, 4) if (kb >> s) >= 1]
    names += [f"bs_128x128_k{s}" for s in range(0, 4) if (kb >> s) >= 2]
    if M > 128:
        names += ["bs_256x256", "bs_256x128"]
    return names


def candidates(M: int, N: int, K: int, family: str):
    """(pair, swap, bn, stages, log2_splitk) tuples worth timing for this shape."""
    if family.startswith("a8w8_blockscale"):
        return blockscale_candidates(M, N, K)
    elems = {"bf16": 64, "a4w4": 256}.get(family, 128)
    k_iters = max(1, (K + elems - 1) // elems)
    out = []
    splits = [s for s in range(0, 6) if (k_iters >> s) >= 2] or [0]
    if M <= 256:
        for bn in (16, 32, 64, 128, 256):
            if bn < M or (bn >= 2 * max(M, 16) and bn > 16):
                continue
            if bn <= 64:
                # decode kernel: its own stage count (two CTAs per SM) or three stages, K split over a cluster of up to 4
                for st in (0, 3):
                    for sk in [s for s in splits if s <= 2]:
                        out.append((0, 1, bn, st, sk))
                for sk in [s for s in splits if s > 2]:
                    out.append((0, 1, bn, 4, sk))
                continue
            for st in (4, 8):
                for sk in splits:
                    out.append((0, 1, bn, st, sk))
    if 64 < M <= 256:
        # the decode kernel on up to four tiles of 64 (or two of 128) activation rows, each streaming the same weight tile
        for st in (0, 3):
            for sk in [s for s in splits if s <= 2]:
                out.append((0, 1, 64, st, sk))
            for sk in [s for s in splits if s <= 1]:
                out.append((0, 1, 128, st, sk))
    if M >= 64:
        for pair in (0, 1):
            for bn in (64, 128, 192, 224, 256):
                if pair and (M < 512 or bn < 128):
                    continue
                if bn > 128 and N % bn and N % 128 == 0 and bn not in (256,):
                    pass  # ragged last tile is allowed, just less efficient
                for sk in ([0] if M >= 2048 else splits[:4]):
                    out.append((pair, 0, bn, 0, sk))
    return out


# --------------------------------------------------------------------------------------- problems
def _rand_u8(lo, hi, *shape, device):
    return torch.randint(lo, hi, shape, dtype=torch.uint8, device=device)


def _rand_e4m3(rows, cols, device):
    """Signed e4m3 values of magnitude 2^-3 .. 2, so that long sums stay inside the fp32 reference's accuracy."""
    mag = _rand_u8(0x20, 0x40, rows, cols, device=device)
    return (mag | (_rand_u8(0, 2, rows, cols, device=device) << 7)).view(torch.float8_e4m3fn)


def make_problem(family: str, M: int, N: int, K: int, device, seed: int):
    """-> (args for the entry point, reference fp32 output of the first `ref_rows` rows, ref_rows)."""
    torch.manual_seed(seed)
    ref_rows = min(M, 256)
    if family == "bf16":
        a = (torch.randn(M, K, device=device) * 0.1).to(torch.bfloat16)
        b = (torch.randn(N, K, device=device) * 0.1).to(torch.bfloat16)
        ref = a[:ref_rows].float() @ b.float().T
        return (a, b), ref, ref_rows
    if family.startswith("a8w8_blockscale"):
        a, b = _rand_e4m3(M, K, device), _rand_e4m3(N, K, device)
        xs = torch.rand(M, K // 128, device=device) + 0.5
        ws = torch.rand((N + 127) // 128, K // 128, device=device) + 0.5
        ref = (a[:ref_rows].float() * xs[:ref_rows].repeat_interleave(128, dim=1)) @ (
            b.float() * ws.repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)).T
        out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        if family.endswith("bpreshuffle"):
            # the pre-shuffled-weight form: (16,16)-shuffled weight, x_scale stored K-block-major under an [M, K/128] view
            return (a, shuffle.shuffle_weight(b), xs.T.contiguous().view(M, K // 128), ws, out), ref, ref_rows
        return (a, b, xs, ws, out), ref, ref_rows
    sa = _rand_u8(125, 129, M, K // 32, device=device)
    sb = _rand_u8(125, 129, N, K // 32, device=device)
    sa_f = fp4_utils.e8m0_to_f32(sa[:ref_rows]).repeat_interleave(32, dim=1)
    sb_f = fp4_utils.e8m0_to_f32(sb).repeat_interleave(32, dim=1)
    if family == "a4w4":
        a, b = _rand_u8(0, 256, M, K // 2, device=device), _rand_u8(0, 256, N, K // 2, device=device)
        ref = (fp4_utils.mxfp4_to_f32(a[:ref_rows]) * sa_f) @ (fp4_utils.mxfp4_to_f32(b) * sb_f).T
        out = torch.empty(((M + 31) // 32 * 32, N), dtype=torch.bfloat16, device=device)
        return (a, shuffle.shuffle_weight(b), shuffle.shuffle_scale(sa), shuffle.shuffle_scale(sb), out), ref, ref_rows
    a = _rand_e4m3(M, K, device)
    if family == "a8w8_mxfp8":
        b = _rand_e4m3(N, K, device)
        ref = (a[:ref_rows].float() * sa_f) @ (b.float() * sb_f).T
    else:
        b = _rand_u8(0, 256, N, K // 2, device=device)
        ref = (a[:ref_rows].float() * sa_f) @ (fp4_utils.mxfp4_to_f32(b) * sb_f).T
    out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    return (a, shuffle.shuffle_mxfp8fp4_b(b), shuffle.shuffle_mxfp8fp4_scale(sa), shuffle.shuffle_mxfp8fp4_scale(sb), out), ref, ref_rows


def run_candidate(family: str, args, cand):
    if family.startswith("a8w8_blockscale"):
        a, b, xs, ws, out = args
        _ffi.call("gemm_a8w8_blockscale_bpreshuffle" if family.endswith("bpreshuffle") else "gemm_a8w8_blockscale", a, b, xs, ws, out, 0, cand or None)
        return out
    pair, swap, bn, st, sk = cand
    kid = kernel_id(pair, swap, bn, st)
    if family == "bf16":
        a, b = args
        y = torch.empty((1, a.shape[0], b.shape[0]), dtype=torch.bfloat16, device=a.device)
        _ffi.call("opus_gemm_a16w16_tune", a[None], b[None], y, None, kid, sk)
        return y[0]
    if family == "a4w4":
        a, b, sa, sb, out = args
        _ffi.call("gemm_a4w4_blockscale_tune", a, b, sa, sb, out, kid, sk)
        return out[: a.shape[0]]
    a, b, sa, sb, out = args
    # these entry points take only a kernel name: the K split travels as its "_k<n>" suffix
    fn = "mxfp8_mxfp8_gemm_asm" if family == "a8w8_mxfp8" else "mxfp8_mxfp4_gemm_asm"
    _ffi.call(fn, a, b, sa, sb, out, kernel_name(pair, swap, bn, st, sk), 0)
    return out


def err_ratio(ref: torch.Tensor, out: torch.Tensor, rows: int, rtol=1e-2, atol=1e-2) -> float:
    o = out[:rows].float()
    bad = ~((ref - o).abs() <= atol + rtol * o.abs())
    return float(bad.float().mean().item())


def time_candidate(family, arg_sets, cand, iters=20) -> float:
    """Device microseconds per call, CUDA-graph replay over rotating argument sets."""
    n = len(arg_sets)
    s = _side_stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(max(3, n)):
            run_candidate(family, arg_sets[i % n], cand)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                run_candidate(family, arg_sets[i % n], cand)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


_STREAM = None


def _side_stream():
    """One capture stream for the whole run: the library keeps a split-K workspace per stream."""
    global _STREAM
    if _STREAM is None:
        _STREAM = torch.cuda.Stream()
    return _STREAM


def bytes_of(family, M, N, K):
    bpe = {"bf16": (2, 2), "a4w4": (0.5, 0.5), "a8w8_mxfp8": (1, 1), "a8w4_mxfp8": (1, 0.5)}.get(family, (1, 1))
    return int(M * K * bpe[0] + N * K * bpe[1] + 2 * M * N)  # scale bytes not counted, as in the reference's `bw`


def tune_shape(family, M, N, K, device, verbose=False):
    problem_bytes = bytes_of(family, M, N, K)
    n_sets = max(2, min(8, int(2.2 * 126e6 // max(problem_bytes, 1)) + 1))
    sets, ref, rows = [], None, 0
    for i in range(n_sets):
        args, r, rows_i = make_problem(family, M, N, K, device, seed=i)
        sets.append(args)
        if i == 0:
            ref, rows = r, rows_i
    best = None
    for cand in candidates(M, N, K, family):
        try:
            out = run_candidate(family, sets[0], cand)
            torch.cuda.synchronize()
            if _ffi.device_status(device.index or 0) != (0, 0, 0, 0):
                continue
            err = err_ratio(ref, out, rows)
            if err > 0.0:
                if verbose:
                    print(f"  {cand}: rejected, errRatio {err:.4f}", file=sys.stderr)
                continue
            us = time_candidate(family, sets, cand)
        except RuntimeError as e:
            if verbose:
                print(f"  {cand}: {str(e)[:100]}", file=sys.stderr)
            continue
        if verbose:
            print(f"  {cand}: {us:.2f} us", file=sys.stderr)
        if best is None or us < best[1]:
            best = (cand, us, err)
    return best


def write_rows(path, family, rows):
    header = BF16_HEADER if family == "bf16" else (BLOCKSCALE_HEADER if family.startswith("a8w8_blockscale") else HEADER)
    tmp = path + ".tmp"
    with open(tmp, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=header, lineterminator="\n")
        w.writeheader()
        for key in sorted(rows):
            w.writerow(rows[key])
    os.replace(tmp, path)


def read_rows(path, family):
    rows = {}
    if os.path.exists(path):
        with open(path, newline="") as f:
            for r in csv.DictReader(f):
                if r.get("M"):
                    rows[(r["gfx"], int(r["cu_num"]), int(r["M"]), int(r["N"]), int(r["K"]))] = r
    return rows


def shapes_from_file(path):
    """(M, N, K) of every row of a CSV with M, N, K columns (an untuned-shape list such as the one tgemm.mm records with
    AITER_TUNE_GEMM=1, or a tuned table)."""
    out = []
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            if r.get("M"):
                shape = (int(r["M"]), int(r["N"]), int(r["K"]))
                if shape not in out:
                    out.append(shape)
    return out


def _family_tables(family):
    from . import gemm_op_a4w4, gemm_op_a8w4, gemm_op_a8w8, gemm_op_a16w16

    return {"a4w4": [gemm_op_a4w4._table], "a8w8_mxfp8": [gemm_op_a8w8._mxfp8_table], "a8w4_mxfp8": [gemm_op_a8w4._table],
            "bf16": [gemm_op_a16w16._bf16_table], "a8w8_blockscale": [gemm_op_a8w8._blockscale_table],
            "a8w8_blockscale_bpreshuffle": [gemm_op_a8w8._blockscale_bpreshuffle_table]}[family]


def use_table(family, path):
    """Point the family's AITER_CONFIG_GEMM_* variable at `path` (None: the packaged table) and drop the cached rows."""
    env = config.TABLES[FAMILIES[family][0]][0]
    if path is None:
        os.environ.pop(env, None)
    else:
        os.environ[env] = path
    for t in _family_tables(family):
        t.clear()


def run_production(family, args):
    """The call a user of the library makes, with whatever the tables say for this shape."""
    from . import gemm_op_a4w4, gemm_op_a8w4, gemm_op_a8w8, tuned_gemm

    if family == "bf16":
        return tuned_gemm.tgemm.mm(args[0], args[1])
    if family == "a4w4":
        a, b, sa, sb, _ = args
        return gemm_op_a4w4.gemm_a4w4(a, b, sa, sb)
    a, b, sa, sb, _ = args
    if family == "a8w8_mxfp8":
        return gemm_op_a8w8.gemm_a8w8_mxfp8(a, b, sa, sb, a_preshuffle=False)
    if family == "a8w4_mxfp8":
        return gemm_op_a8w4.gemm_a8w4_mxfp8(a, b, sa, sb, a_preshuffle=False)
    if family == "a8w8_blockscale":
        return gemm_op_a8w8.gemm_a8w8_blockscale(a, b, sa, sb)
    return gemm_op_a8w8.gemm_a8w8_blockscale_bpreshuffle(a, b, sa, sb)


def run_config(family, shapes, device, table_path=None, verbose=True):
    """Time the production operator for every shape (aiter/utility/base_tuner.py:571-583): -> {shape: us, or None when the
    call failed or missed the tolerance}.  `table_path` names the tuned table to use (None: the packaged one)."""
    use_table(family, table_path)
    results = {}
    for (M, N, K) in shapes:
        try:
            problem_bytes = bytes_of(family, M, N, K)
            n_sets = max(2, min(8, int(2.2 * 126e6 // max(problem_bytes, 1)) + 1))
            sets = [make_problem(family, M, N, K, device, seed=i) for i in range(n_sets)]
            out = run_production(family, sets[0][0])
            torch.cuda.synchronize()
            ok = _ffi.device_status(device.index or 0) == (0, 0, 0, 0) and err_ratio(sets[0][1], out, sets[0][2]) == 0.0
            us = time_production(family, [t[0] for t in sets]) if ok else None
        except RuntimeError as e:
            us = None
            if verbose:
                print(f"  {family} {M}x{N}x{K}: {str(e)[:120]}", file=sys.stderr)
        results[(M, N, K)] = us
        if verbose:
            print(f"{family} {M}x{N}x{K}: " + ("failed" if us is None else f"{us:.2f} us  {2.0 * M * N * K / us / 1e6:.2f} TFLOPS"))
    return results


def time_production(family, arg_sets, iters=20):
    n = len(arg_sets)
    s = _side_stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(max(3, n)):
            run_production(family, arg_sets[i % n])
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                run_production(family, arg_sets[i % n])
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def make_row(family, gfx, cu, M, N, K, best):
    cand, us, err = best
    tflops = round(2.0 * M * N * K / us / 1e6, 2)
    bw = round(bytes_of(family, M, N, K) / us / 1e3, 2)
    row = {"gfx": gfx, "cu_num": cu, "M": M, "N": N, "K": K, "us": round(us, 4), "tflops": tflops, "bw": bw}
    if family.startswith("a8w8_blockscale"):
        base = cand.split("_k")[0] if cand else ""
        row.update({"libtype": "b200", "kernelId": BLOCKSCALE_VARIANTS.get(base, 0), "splitK": int(cand.split("_k")[1]) if "_k" in cand else 0,
                    "kernelName": cand, "errRatio": err})
        return row, cand or "(launcher's model)"
    pair, swap, bn, st, sk = cand
    name = kernel_name(pair, swap, bn, st) if family in ("a4w4", "bf16") else kernel_name(pair, swap, bn, st, sk)
    row.update({"splitK": sk, "kernelName": name})
    if family == "bf16":
        row.update({"bias": False, "dtype": "torch.bfloat16", "outdtype": "torch.bfloat16", "scaleAB": False,
                    "bpreshuffle": False, "libtype": "opus", "solidx": kernel_id(pair, swap, bn, st), "err_ratio": err})
    else:
        row.update({"kernelId": kernel_id(pair, swap, bn, st), "errRatio": err})
    return row, f"{name} splitK 2^{sk}"


# --------------------------------------------------------------------------------------- worker pool (one process per GPU)
def worker_command(family, shapes, part_path, gpu, args):
    """Command line of one worker: this tuner on a subset of the shapes, one GPU, its own output file."""
    cmd = os.environ.get("AITER_B200_TUNE_WORKER_CMD")  # tests substitute a stand-in that needs no GPU
    base = cmd.split() if cmd else [sys.executable, "-m", "aiter_b200.tune"]
    out = base + ["--family", family, "--shapes", ";".join(",".join(str(v) for v in s) for s in shapes), "-o", part_path, "--retune"]
    if args.verbose:
        out.append("-v")
    return out, dict(os.environ, CUDA_VISIBLE_DEVICES=str(gpu))


def run_pool(family, shapes, n_workers, timeout_s, args, poll_s=0.2):
    """Spread `shapes` over `n_workers` worker processes (worker i on GPU i).  A worker that exits non-zero or outlives
    `timeout_s` is killed (only that process) and its shapes not yet written go to a fresh worker once; what fails twice
    is reported.  -> (rows by key, failed shapes)."""
    tmpdir = tempfile.mkdtemp(prefix="aiter_b200_tune_")
    pending = [(list(shapes[i::n_workers]), i, 0) for i in range(n_workers) if shapes[i::n_workers]]
    running, rows, failed, serial = [], {}, [], 0
    while pending or running:
        while pending and len(running) < n_workers:
            todo, gpu, attempt = pending.pop(0)
            serial += 1
            part = os.path.join(tmpdir, f"part{serial}.csv")
            cmd, env = worker_command(family, todo, part, gpu, args)
            proc = subprocess.Popen(cmd, env=env, stdout=subprocess.DEVNULL if not args.verbose else None, stderr=subprocess.STDOUT if not args.verbose else None)
            running.append({"proc": proc, "todo": todo, "gpu": gpu, "attempt": attempt, "part": part, "t0": time.time()})
        time.sleep(poll_s)
        for w in list(running):
            rc = w["proc"].poll()
            timed_out = rc is None and time.time() - w["t0"] > timeout_s
            if rc is None and not timed_out:
                continue
            if timed_out:
                w["proc"].kill()  # this worker only: by its own handle, never by pattern
                w["proc"].wait()
            running.remove(w)
            done = read_rows(w["part"], family)
            rows.update(done)
            left = [s for s in w["todo"] if not any(k[2:] == s for k in done)]
            if left and (rc != 0 or timed_out):
                what = "ran out of time" if timed_out else f"exited with code {rc}"
                if w["attempt"] == 0:
                    print(f"worker on GPU {w['gpu']} {what}; {len(left)} shape(s) go to another worker")
                    pending.append((left, (w["gpu"] + 1) % n_workers, 1))
                else:
                    print(f"worker on GPU {w['gpu']} {what} again; giving up on {left}")
                    failed += left
            elif left:
                failed += left  # the worker ran to its end and found no valid candidate
    return rows, failed


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", choices=sorted(FAMILIES), required=True)
    ap.add_argument("--shapes", default="", help='"M,N,K;M,N,K;..."')
    ap.add_argument("-i", "--untune_file", default=None, help="CSV with M,N,K columns: the shapes to tune (e.g. the list tgemm.mm records)")
    ap.add_argument("--baseline", action="store_true", help="tune the benchmark shapes of this family")
    ap.add_argument("-o", "--output", default=None, help="CSV to update (default: the packaged table)")
    ap.add_argument("--retune", action="store_true", help="re-measure shapes already in the file")
    ap.add_argument("--run_config", nargs="?", const=True, default=False, metavar="TUNED_CSV",
                    help="time the production operator and exit (no tuning); with a CSV: its shapes and its kernels")
    ap.add_argument("--compare", action="store_true", help="time the production operator before and after tuning and print both")
    ap.add_argument("--update_improved", action="store_true", help="with --compare: write only the rows that improved by --min_improvement_pct")
    ap.add_argument("--min_improvement_pct", type=float, default=3.0)
    ap.add_argument("--mp", type=int, default=1, help="worker processes, one per GPU")
    ap.add_argument("--timeout", type=int, default=1800, help="seconds a worker may run before it is killed and its shapes re-queued")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args(argv)
    if args.update_improved and not args.compare:
        ap.error("--update_improved requires --compare")
    table, _ = FAMILIES[args.family]
    path = args.output or os.path.join(config.CONFIG_DIR, config.TABLES[table][1])
    shapes = [tuple(int(v) for v in s.split(",")) for s in args.shapes.split(";") if s.strip()]
    if args.untune_file:
        shapes += shapes_from_file(args.untune_file)
    if args.baseline:
        shapes += BASELINE_SHAPES[args.family]
    if isinstance(args.run_config, str) and not shapes:
        shapes = shapes_from_file(args.run_config)
    gfx, cu = config.get_gfx(), config.get_cu_num()

    if args.mp > 1 and not args.run_config:
        rows = read_rows(path, args.family)
        todo = [s for s in shapes if args.retune or (gfx, cu) + s not in rows]
        new_rows, failed = run_pool(args.family, todo, args.mp, args.timeout, args)
        rows.update(new_rows)
        write_rows(path, args.family, rows)
        print(f"{args.family}: {len(new_rows)} shape(s) tuned by {args.mp} workers, {len(failed)} failed{': ' + str(failed) if failed else ''}")
        return 1 if failed else 0

    if not torch.cuda.is_available():
        raise SystemExit("the tuner measures on the GPU: no CUDA device found")
    device = torch.device("cuda", torch.cuda.current_device())
    if args.run_config:
        res = run_config(args.family, shapes, device, args.run_config if isinstance(args.run_config, str) else None)
        return 0 if all(v is not None for v in res.values()) else 1

    before = run_config(args.family, shapes, device, path if os.path.exists(path) else None, verbose=False) if args.compare else {}
    rows = read_rows(path, args.family)
    candidate_rows = dict(rows)
    tuned = []
    for (M, N, K) in shapes:
        key = (gfx, cu, M, N, K)
        if key in rows and not args.retune and not args.compare:
            print(f"{args.family} {M}x{N}x{K}: already tuned, skipped")
            continue
        best = tune_shape(args.family, M, N, K, device, args.verbose)
        if best is None:
            print(f"{args.family} {M}x{N}x{K}: no valid candidate")
            continue
        row, text = make_row(args.family, gfx, cu, M, N, K, best)
        candidate_rows[key] = row
        tuned.append((M, N, K))
        if not args.compare:
            rows[key] = row
            write_rows(path, args.family, rows)
        print(f"{args.family} {M}x{N}x{K}: {text}  {best[1]:.2f} us  {row['tflops']} TFLOPS  {row['bw']} GB/s")
    if args.compare:
        cand_path = path + ".compare_candidate.csv"
        write_rows(cand_path, args.family, candidate_rows)
        after = run_config(args.family, tuned, device, cand_path, verbose=False)
        use_table(args.family, None)
        kept = 0
        for shape in tuned:
            b, a = before.get(shape), after.get(shape)
            gain = None if (a is None or b is None) else (b - a) / b * 100.0
            improved = a is not None and (b is None or gain >= args.min_improvement_pct)
            print(f"{args.family} {shape[0]}x{shape[1]}x{shape[2]}: before {'-' if b is None else f'{b:.2f} us'}  after {'-' if a is None else f'{a:.2f} us'}"
                  f"  {'' if gain is None else f'{gain:+.1f} %'}  {'improved' if improved else 'kept'}")
            if args.update_improved and improved:
                rows[(gfx, cu) + shape] = candidate_rows[(gfx, cu) + shape]
                kept += 1
        if args.update_improved:
            write_rows(path, args.family, rows)
            print(f"{kept} of {len(tuned)} rows updated in {path}; all candidates kept in {cand_path}")
        else:
            print(f"candidates written to {cand_path}; {path} left unchanged (no --update_improved)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
