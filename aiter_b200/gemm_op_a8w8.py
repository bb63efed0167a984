"""MXFP8 x MXFP8 GEMM (reference: aiter/ops/gemm_op_a8w8.py:1215-1254) with table-driven dispatch."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _ffi, dtypes
from .config import TunedTable

_mxfp8_table = TunedTable("a8w8_mxfp8")


def get_MXFP8_config(M: int, N: int, K: int):
    return _mxfp8_table.lookup(M, N, K)


def gemm_a8w8_mxfp8(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, dtype: torch.dtype = dtypes.bf16,
                    a_preshuffle: bool = True, kernelName: str = "") -> Tensor:
    """D[M,N] bf16 = A @ B^T, A/B e4m3 with e8m0 scales per 32 along K.  A is (m/2,k/128,2,128)-tiled when
    a_preshuffle, B is always 16x16-byte tile transposed, scales are in the (m/32,k/4,32,4) layout."""
    M, N = A.shape[0], B.shape[0]
    out = torch.empty((M, N), dtype=dtype, device=A.device)
    if not kernelName:
        cfg = get_MXFP8_config(M, N, A.shape[1])
        if cfg is not None:
            kernelName = cfg.get("kernelName") or ""
    _ffi.call("mxfp8_mxfp8_gemm_asm", A, B, ScaleA, ScaleB, out, kernelName if kernelName else None, int(bool(a_preshuffle)))
    return out
