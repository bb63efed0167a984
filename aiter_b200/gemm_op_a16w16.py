"""bf16 GEMM wrappers (reference: aiter/ops/gemm_op_a16w16.py:12-76, aiter/ops/opus/gemm_op_a16w16.py:88-238,448-540)."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _ffi
from .config import TunedTable

_bf16_table = TunedTable("bf16", extra_keys=("bias", "dtype", "outdtype", "scaleAB", "bpreshuffle"))


def gemm_a16w16_asm(A: Tensor, B: Tensor, out: Tensor, bias: Tensor | None = None, splitK: int | None = None,
                    kernelName: str | None = None, bpreshuffle: bool = False) -> Tensor:
    """out[M,N] = A[M,K] @ B[N,K]^T (+ bias[N]).  The reference passes a per-stream semaphore tensor for its
    split-K tickets; here the tickets live in the library's per-stream workspace, so none is needed."""
    _ffi.call("gemm_a16w16_asm", A, B, out, None, bias, splitK, kernelName if kernelName else None, int(bool(bpreshuffle)))
    return out


def _check_a16w16_tune_layout(XQ: Tensor, WQ: Tensor, Y: Tensor):
    """Reject layouts the launcher cannot serve (same rules as the reference's guard)."""
    for name, t in (("XQ", XQ), ("WQ", WQ), ("Y", Y)):
        if t.dim() != 3:
            raise ValueError(f"opus_gemm_a16w16_tune: {name} must be 3D (got {name}.shape={tuple(t.shape)}).")
    batch, M, K = XQ.shape
    b_w, N, K_w = WQ.shape
    if (b_w, K_w) != (batch, K):
        raise ValueError(f"opus_gemm_a16w16_tune: WQ shape mismatch (got WQ.shape={tuple(WQ.shape)}, expected ({batch}, N, {K})); XQ.shape={tuple(XQ.shape)}")
    if tuple(Y.shape) != (batch, M, N):
        raise ValueError(f"opus_gemm_a16w16_tune: Y shape mismatch (got Y.shape={tuple(Y.shape)}, expected ({batch}, {M}, {N}))")
    for name, t, rows in (("XQ", XQ, M), ("WQ", WQ, N)):
        s0, s1, s2 = t.stride()
        if not (s2 == 1 and s1 >= t.shape[2] and (batch == 1 or s0 == rows * s1)):
            raise NotImplementedError(
                f"opus_gemm_a16w16_tune: {name} must be K-contiguous with an optional padded leading dim "
                f"(got {name}.stride()={tuple(t.stride())}, {name}.shape={tuple(t.shape)}); materialize with `.contiguous()`."
            )
    if tuple(Y.stride()) != (M * N, N, 1):
        raise NotImplementedError(f"opus_gemm_a16w16_tune: Y must have contiguous strides {(M * N, N, 1)} (got {tuple(Y.stride())}).")


def opus_gemm_a16w16_tune(XQ: Tensor, WQ: Tensor, Y: Tensor, bias=None, kernelId: int = 0, splitK: int = 0) -> Tensor:
    """Id-based dispatcher: Y[b,M,N] = XQ[b,M,K] @ WQ[b,N,K]^T.  `kernelId` indexes the kernel menu
    (aiter_b200.kernel_list()), `splitK` is log2 of the K split.  The old positional form
    (XQ, WQ, Y, kernelId, splitK) is still accepted."""
    if isinstance(bias, int) and not isinstance(bias, bool):
        kernelId, splitK, bias = bias, (splitK if (splitK != 0 and kernelId == 0) else kernelId), None
    _check_a16w16_tune_layout(XQ, WQ, Y)
    _ffi.call("opus_gemm_a16w16_tune", XQ, WQ, Y, bias, kernelId, splitK)
    return Y


def opus_gemm(XQ: Tensor, WQ: Tensor, Y: Tensor, group_layout=None, x_scale=None, w_scale=None, bias=None) -> Tensor:
    """Y[b,M,N] = XQ[b,M,K] @ WQ[b,N,K]^T in one launch.  bf16 operands: Y bf16 or fp32, optional bias [N] or [b,N].
    fp8 operands with x_scale [b,M,K/128] and w_scale [b,N/128,K/128] (fp32): the 128-block-scaled product, Y fp32
    (the reference's a8w8_scale pipeline, csrc/opus_gemm/opus_gemm.cu:153-186)."""
    _ffi.call("opus_gemm", XQ, WQ, Y, group_layout, x_scale, w_scale, bias)
    return Y


def gemm_a16w16_opus(A: Tensor, B: Tensor, bias: Tensor | None = None, dtype: torch.dtype = torch.bfloat16,
                     out: Tensor | None = None) -> Tensor:
    """Shape-driven bf16 GEMM: rows of the bf16 table with libtype 'opus' choose (kernelId, splitK);
    other shapes go through the library heuristic.  A [M,K] or [b,M,K]; B [N,K] or [b,N,K]."""
    if A.dtype != torch.bfloat16 or B.dtype != torch.bfloat16:
        raise NotImplementedError(f"gemm_a16w16_opus only supports bf16 A/B (got A.dtype={A.dtype}, B.dtype={B.dtype}).")
    if dtype not in (torch.bfloat16, torch.float32):
        raise NotImplementedError(f"gemm_a16w16_opus only supports bf16/fp32 output dtype, got {dtype}")
    squeeze = A.dim() == 2
    A3 = A.unsqueeze(0) if squeeze else A
    B3 = B.unsqueeze(0) if B.dim() == 2 else B
    batch, M, K = A3.shape
    N = B3.shape[1]
    if out is None:
        out = torch.empty((batch, M, N), dtype=dtype, device=A.device)
    Y3 = out.unsqueeze(0) if out.dim() == 2 else out
    cfg = _bf16_table.lookup(M, N, K, bias is not None, str(A.dtype), str(dtype), False, False)
    if cfg is not None and cfg.get("libtype") == "opus":
        opus_gemm_a16w16_tune(A3, B3, Y3, bias, int(cfg.get("solidx") or 0), int(cfg.get("splitK") or 0))
    else:
        opus_gemm(A3, B3, Y3, None, None, None, bias)
    return out.squeeze(0) if (squeeze and out.dim() == 3) else out
