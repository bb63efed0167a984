"""MXFP4 x MXFP4 GEMM entry points (reference: aiter/ops/gemm_op_a4w4.py:33-78,147-287,581-608)."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _ffi, dtypes
from .config import TunedTable

_table = TunedTable("a4w4")


def get_GEMM_config(M: int, N: int, K: int):
    """Tuned row for (M, N, K): exact M, then the padded-M buckets; None when the shape is untuned."""
    return _table.lookup(M, N, K)


def gemm_a4w4_asm(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, out: Tensor, kernelName: str = "",
                  bias: Tensor | None = None, alpha: float | None = 1.0, beta: float | None = 0.0,
                  bpreshuffle: bool | None = True, log2_k_split: int | None = None) -> Tensor:
    """out[:M] = alpha * A.B^T + beta * bias.  A [M,K/2], B [N,K/2] packed e2m1 (B (16,16)-shuffled when
    bpreshuffle), scales e8m0 in the e8m0_shuffle layout, out [>=M, N] bf16."""
    _ffi.call(
        "gemm_a4w4_asm", A, B, A_scale, B_scale, out, kernelName if kernelName else None, bias,
        alpha if alpha is not None else 1.0, beta if beta is not None else 0.0,
        int(bpreshuffle) if bpreshuffle is not None else 1,
        log2_k_split if log2_k_split is not None else -1,
    )
    return out


def gemm_a4w4_blockscale(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, Out: Tensor, splitK: int = 0,
                         kernelName: str = "") -> Tensor:
    _ffi.call("gemm_a4w4_blockscale", XQ, WQ, x_scale, w_scale, Out, splitK, kernelName if kernelName else None)
    return Out


def gemm_a4w4_blockscale_tune(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, Out: Tensor, kernelId: int = 0,
                              splitK: int = 0) -> Tensor:
    _ffi.call("gemm_a4w4_blockscale_tune", XQ, WQ, x_scale, w_scale, Out, kernelId, splitK)
    return Out


def gemm_mxfp4_asm(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, dtype: torch.dtype = dtypes.bf16,
                   a_preshuffle: bool = False, kernelName: str = "") -> Tensor:
    """MXFP4 GEMM with the (m/32,k/4,32,4) scale layout and a 16x16-byte tiled B (aiter/ops/gemm_op_a4w4.py:290-330)."""
    if dtype != dtypes.bf16:
        raise NotImplementedError("gemm_mxfp4_asm: only bf16 output is built")
    out = torch.empty((A.shape[0], B.shape[0]), dtype=dtype, device=A.device)
    _ffi.call("mxfp4_gemm_asm", A, B, ScaleA, ScaleB, out, None, kernelName if kernelName else None, int(bool(a_preshuffle)))
    return out


def gemm_a4w4(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, bias: Tensor | None = None,
              dtype: torch.dtype = dtypes.bf16, alpha: float | None = 1.0, beta: float | None = 0.0,
              bpreshuffle: bool | None = True, apreshuffle: bool | None = False,
              global_A_scale: Tensor | None = None, global_B_scale: Tensor | None = None) -> Tensor:
    """A4W4 GEMM returning one bf16 tensor [.., N].  The tuned table chooses the kernel and split-K for
    (M, N, K); untuned shapes use the library heuristic."""
    if dtype in (dtypes.fp4x2, dtypes.fp8):
        raise NotImplementedError("gemm_a4w4 returns one plain-dtype tensor; use gemm_a4w4o4 / gemm_a4w4o8")
    if global_A_scale is not None or global_B_scale is not None:
        raise NotImplementedError("NVFP4 (per-tensor global scales) is not built")
    m = A.numel() // A.shape[-1]
    n = B.shape[0]
    k = A.shape[-1] * 2
    out = torch.empty(((m + 31) // 32 * 32, n), dtype=dtype, device=A.device)
    cfg = get_GEMM_config(m, n, k)
    splitK, kernelName = None, ""
    if cfg is not None:
        splitK = cfg.get("splitK")
        kernelName = cfg.get("kernelName") or ""
    gemm_a4w4_asm(A.view(m, k // 2), B, A_scale, B_scale, out, kernelName, bias, alpha, beta, bpreshuffle, log2_k_split=splitK)
    return out[:m].view(*A.shape[:-1], n)
