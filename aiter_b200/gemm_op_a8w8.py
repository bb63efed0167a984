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


def gemm_a8w8_mxfp8_noalloc(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, out: Tensor, a_preshuffle: bool = True,
                            log2_k_split: int | None = None) -> Tensor:
    """Same GEMM as gemm_a8w8_mxfp8, for callers that may not allocate device memory: `out` [M,N] bf16 is
    supplied by the caller, and the library keeps its split-K partial sums, tickets and status record in a
    fixed 8 MiB + 32 KiB array that is part of its image instead of cudaMalloc'ing them.  Think of a server
    that gave all memory to one arena at start-up, or a plugin that must not touch its host's allocator.
    Shapes whose split-K scratch would not fit raise RuntimeError.  Make the first call on a device before any
    CUDA-graph capture; calls that overlap on the GPU share (and race on) the one array."""
    _ffi.call("aiter_b200_gemm_a8w8_mxfp8_noalloc", A, B, ScaleA, ScaleB, out, int(bool(a_preshuffle)),
              -1 if log2_k_split is None else int(log2_k_split))
    return out
