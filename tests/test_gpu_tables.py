"""Every row of every committed tuned table, at its own (M, N, K): the public operator is called so that the table
picks the row's kernel and K split, and up to 64 random rows of the output (all N columns) are compared with the
numpy oracle.  Inputs are seeded bf16 N(0,1) data quantised on the GPU by the torch quantisers (which
tests/test_gpu_quant.py pins byte for byte to their CPU form, and the CPU tests pin to the oracle); the quantised
bytes are copied back for the oracle, so both sides see the same operands."""
import csv
import os

import numpy as np
import pytest
import torch

from helpers import check
from oracle import mx_oracle as ox

pytestmark = pytest.mark.gpu

CONFIG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "aiter_b200", "configs")
FILES = {
    "a4w4": "a4w4_blockscale_tuned_gemm.csv",
    "a8w8_mxfp8": "a8w8_mxfp8_tuned_gemm.csv",
    "a8w4_mxfp8": "a8w4_mxfp8_tuned_gemm.csv",
    "bf16": "bf16_tuned_gemm.csv",
    "a8w8_blockscale": "a8w8_blockscale_tuned_gemm.csv",
    "a8w8_blockscale_bpreshuffle": "a8w8_blockscale_bpreshuffle_tuned_gemm.csv",
}


def _rows():
    out = []
    for family, name in FILES.items():
        with open(os.path.join(CONFIG_DIR, name), newline="") as f:
            for r in csv.DictReader(f):
                out.append((family, int(r["M"]), int(r["N"]), int(r["K"]), r["kernelName"] or "", int(float(r["splitK"] or 0))))
    # rows that share a weight run back to back, so the weight is quantised and dequantised once
    return sorted(out, key=lambda t: (t[0], t[2], t[3], t[1]))


ROWS = _rows()


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def _randn(rows, cols, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(rows, cols, generator=g, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


_weight_cache = {}


def _weight(ab, family, N, K):
    """-> (device operands of the weight in wire layout, fp32 dequantised weight on the CPU); one entry is kept."""
    key = (family, N, K)
    if key not in _weight_cache:
        _weight_cache.clear()
        w = _randn(N, K, 2, 0.1 if family == "bf16" else 1.0)
        if family == "bf16":
            dev = (w,)
            deq = w.float().cpu().numpy()
        elif family.startswith("a8w8_blockscale"):
            # e4m3 weight with one fp32 scale per 128 x 128 block
            wq = (w.float() * 2).to(torch.float8_e4m3fn)
            g = torch.Generator(device="cuda").manual_seed(5)
            ws = torch.rand((N + 127) // 128, K // 128, generator=g, device="cuda") + 0.25
            dev = (ab.shuffle_weight(wq, layout=(16, 16)) if family.endswith("bpreshuffle") else wq, ws)
            deq = (ox.e4m3fn_to_f32(wq.view(torch.uint8).cpu().numpy()) *
                   np.repeat(np.repeat(ws.cpu().numpy(), 128, axis=0)[:N], 128, axis=1)).astype(np.float32)
        elif family == "a8w8_mxfp8":
            wq, ws = ab.per_1x32_f8_scale_f8_quant(w, scale_type=ab.dtypes.fp8_e8m0)
            ws = ws.view(torch.uint8)
            dev = (ab.shuffle_mxfp8fp4_b(wq), ab.shuffle_mxfp8fp4_scale(ws))
            deq = ox.dequant_mxfp8(wq.view(torch.uint8).cpu().numpy(), ws.cpu().numpy())
        else:
            wq, ws = ab.per_1x32_f4_quant(w)
            wq, ws = wq.view(torch.uint8), ws.view(torch.uint8)
            if family == "a4w4":
                dev = (ab.shuffle_weight(wq, layout=(16, 16)), ab.fp4_utils.e8m0_shuffle(ws))
            else:
                dev = (ab.shuffle_mxfp8fp4_b(wq), ab.shuffle_mxfp8fp4_scale(ws))
            deq = ox.dequant_mxfp4(wq.cpu().numpy(), ws.cpu().numpy())
        _weight_cache[key] = (dev, deq)
    return _weight_cache[key]


def _table_row(ab, family, M, N, K):
    from aiter_b200 import gemm_op_a4w4, gemm_op_a8w4, gemm_op_a8w8, gemm_op_a16w16

    if family == "a4w4":
        return gemm_op_a4w4.get_GEMM_config(M, N, K)
    if family == "a8w8_mxfp8":
        return gemm_op_a8w8.get_MXFP8_config(M, N, K)
    if family == "a8w4_mxfp8":
        return gemm_op_a8w4.get_A8W4_config(M, N, K)
    if family.startswith("a8w8_blockscale"):
        return gemm_op_a8w8.get_CKGEMM_config(M, N, K, bpreshuffle=family.endswith("bpreshuffle"))
    return gemm_op_a16w16._bf16_table.lookup(M, N, K, False, "torch.bfloat16", "torch.bfloat16", False, False)


@pytest.mark.parametrize("family,M,N,K,kernel,split", ROWS, ids=[f"{r[0]}-{r[1]}x{r[2]}x{r[3]}-{r[4]}" for r in ROWS])
def test_tuned_row(ab, family, M, N, K, kernel, split):
    row = _table_row(ab, family, M, N, K)
    assert row is not None and (row["kernelName"] or "") == kernel, f"the table does not serve ({M},{N},{K}) with {kernel}: {row}"
    dev_w, deq_w = _weight(ab, family, N, K)
    x = _randn(M, K, 1, 0.1 if family == "bf16" else 1.0)
    pick = np.sort(np.random.default_rng(M + N + K).choice(M, size=min(64, M), replace=False))
    launches = ab.launch_count()
    if family == "bf16":
        out = ab.tgemm.mm(x, dev_w[0])
        deq_x = x[pick].float().cpu().numpy()
    elif family.startswith("a8w8_blockscale"):
        xq = (x.float() * 2).to(torch.float8_e4m3fn)
        g = torch.Generator(device="cuda").manual_seed(6)
        xs = torch.rand(M, K // 128, generator=g, device="cuda") + 0.25
        if family.endswith("bpreshuffle"):
            out = ab.gemm_a8w8_blockscale_bpreshuffle(xq, dev_w[0], xs.T.contiguous().view(M, K // 128), dev_w[1])
        else:
            out = ab.gemm_a8w8_blockscale(xq, dev_w[0], xs, dev_w[1])
        deq_x = (ox.e4m3fn_to_f32(xq.view(torch.uint8)[pick].cpu().numpy()) * np.repeat(xs[pick].cpu().numpy(), 128, axis=1)).astype(np.float32)
    elif family == "a4w4":
        xq, xs = ab.per_1x32_f4_quant(x)
        xs = xs.view(torch.uint8)
        out = ab.gemm_a4w4(xq, dev_w[0], ab.fp4_utils.e8m0_shuffle(xs), dev_w[1])
        deq_x = ox.dequant_mxfp4(xq.view(torch.uint8)[pick].cpu().numpy(), xs[pick].cpu().numpy())
    else:
        xq, xs = ab.per_1x32_f8_scale_f8_quant(x, scale_type=ab.dtypes.fp8_e8m0)
        xs = xs.view(torch.uint8)
        fn = ab.gemm_a8w8_mxfp8 if family == "a8w8_mxfp8" else ab.gemm_a8w4_mxfp8
        out = fn(xq, dev_w[0], ab.shuffle_mxfp8fp4_scale(xs), dev_w[1], a_preshuffle=False)
        deq_x = ox.dequant_mxfp8(xq.view(torch.uint8)[pick].cpu().numpy(), xs[pick].cpu().numpy())
    assert out.shape == (M, N)
    assert ab.launch_count() > launches
    ref = ox.f32_to_bf16_bits(ox.gemm_f32(deq_x, deq_w))
    check(ref, out[pick], what=f"{family} ({M},{N},{K}) via table row {kernel} splitK {split}")
    assert ab.device_status(0) == (0, 0, 0, 0)
