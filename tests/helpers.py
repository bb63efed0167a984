"""Seeded problem builders shared by the GPU parity tests.  Inputs are generated on the CPU so the
numpy oracle and the CUDA kernels see identical bytes."""
from __future__ import annotations

import numpy as np
import torch

from oracle import mx_oracle as ox


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def randn_bf16(rows, cols, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * scale).to(torch.bfloat16)


def quant_fp4(x_bf16: torch.Tensor):
    """-> (packed [R,K/2] u8, scales [R,K/32] u8) via the oracle quantiser."""
    q, s = ox.quant_mxfp4(x_bf16.float().numpy())
    return q, s


def quant_fp8(x_bf16: torch.Tensor):
    q, s = ox.quant_mxfp8(x_bf16.float().numpy())
    return q, s


def to_cuda_u8(a: np.ndarray, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.view(dtype) if dtype is not None else t


def check(ref_bits: np.ndarray, out: torch.Tensor, rtol=1e-2, atol=1e-2, what=""):
    """GEMM outputs must be inside rtol = atol = 1e-2 of the oracle on every element."""
    got = bf16_bits(out)
    assert got.shape == ref_bits.shape, f"{what}: shape {got.shape} vs {ref_bits.shape}"
    ratio = ox.mismatch_ratio(ref_bits, got, rtol, atol)
    if ratio != 0.0:
        a = ox.bf16_bits_to_f32(ref_bits).astype(np.float64)
        b = ox.bf16_bits_to_f32(got).astype(np.float64)
        bad = ~(np.abs(a - b) <= atol + rtol * np.abs(b))
        rows = np.unique(np.nonzero(bad)[0])
        cols = np.unique(np.nonzero(bad)[1])
        raise AssertionError(
            f"{what}: {ratio:.4%} of elements outside tolerance; max |diff| {np.nanmax(np.abs(a - b)):.4g}; "
            f"bad rows {rows[:8]}..({len(rows)}), bad cols {cols[:8]}..({len(cols)}); "
            f"ref[0,:4]={a[0, :4]} got[0,:4]={b[0, :4]}"
        )
