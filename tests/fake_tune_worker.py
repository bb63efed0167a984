"""Stand-in for a tuner worker process, for the CPU test of the worker pool: takes the worker's command line, needs no
GPU, and misbehaves on request.  Shapes with M == 13 make the FIRST worker that meets them exit with an error after it
has written its other rows; shapes with M == 17 make the first worker hang; a marker file per shape records that the
first attempt has happened, so the retry succeeds.  M == 19 fails every time."""
import argparse
import csv
import os
import sys
import time

ap = argparse.ArgumentParser()
ap.add_argument("--family")
ap.add_argument("--shapes")
ap.add_argument("-o", "--output")
ap.add_argument("--retune", action="store_true")
ap.add_argument("-v", action="store_true")
a = ap.parse_args()
marks = os.environ["FAKE_WORKER_MARKS"]
header = ["gfx", "cu_num", "M", "N", "K", "kernelId", "splitK", "us", "kernelName", "tflops", "bw", "errRatio"]
rows, misbehave = [], None
for s in a.shapes.split(";"):
    M, N, K = (int(v) for v in s.split(","))
    mark = os.path.join(marks, f"{M}_{N}_{K}")
    first = not os.path.exists(mark)
    open(mark, "a").close()
    if M == 19 or (first and M in (13, 17)):
        misbehave = misbehave or M
        continue
    rows.append({"gfx": "sm_100a", "cu_num": 148, "M": M, "N": N, "K": K, "kernelId": 20, "splitK": 0, "us": 1.0 + M,
                 "kernelName": f"tc5_128x64_n_s0_gpu{os.environ.get('CUDA_VISIBLE_DEVICES', '?')}", "tflops": 1.0, "bw": 1.0, "errRatio": 0.0})
with open(a.output, "w", newline="") as f:
    w = csv.DictWriter(f, fieldnames=header)
    w.writeheader()
    w.writerows(rows)
if misbehave == 17:
    time.sleep(60)
sys.exit(1 if misbehave else 0)
