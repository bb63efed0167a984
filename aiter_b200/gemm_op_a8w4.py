"""MXFP8 activation x MXFP4 weight GEMM (reference: aiter/ops/gemm_op_a8w4.py:18-61) with the
tuned_gemm-style (M,N,K) table the reference lacks on this path."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _ffi, dtypes
from .config import TunedTable

_table = TunedTable("a8w4_mxfp8")


def get_A8W4_config(M: int, N: int, K: int):
    return _table.lookup(M, N, K)


def gemm_a8w4_mxfp8(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, dtype: torch.dtype = dtypes.bf16,
                    a_preshuffle: bool = True, kernelName: str = "") -> Tensor:
    """D[M,N] bf16 = A @ B^T, A [M,K] e4m3, B [N,K/2] packed e2m1, e8m0 scales per 32 on both."""
    M, N = A.shape[0], B.shape[0]
    out = torch.empty((M, N), dtype=dtype, device=A.device)
    if not kernelName:
        cfg = get_A8W4_config(M, N, A.shape[1])
        if cfg is not None:
            kernelName = cfg.get("kernelName") or ""
    _ffi.call("mxfp8_mxfp4_gemm_asm", A, B, ScaleA, ScaleB, out, kernelName if kernelName else None, int(bool(a_preshuffle)))
    return out
