"""Batched bf16 GEMM wrappers (reference: aiter/ops/batched_gemm_op_bf16.py:27-148): Y[b] = XQ[b] @ WQ[b]^T for every
entry of the batch in ONE launch of the persistent kernel (the batch index is one more coordinate of its tile list)."""
from __future__ import annotations

import functools

import torch
from torch import Tensor

from . import _ffi, dtypes
from .config import TunedTable

# (B, M, N, K) -> {kernelId, splitK, kernelName, ...}; the reference keys its table the same way
# (aiter/ops/batched_gemm_op_bf16.py:53-104, AITER_CONFIG_BF16_BATCHED_GEMM)
_batched_table = TunedTable("bf16_batched", extra_keys=("B",))


def batched_gemm_bf16(XQ: Tensor, WQ: Tensor, out: Tensor, bias: Tensor | None = None, splitK: int = 0) -> Tensor:
    """out[b,M,N] = XQ[b,M,K] @ WQ[b,N,K]^T.  As in the reference's CK instances, `bias` is checked (it must have the
    output's dtype) and not added, and `splitK` is accepted and ignored."""
    _ffi.call("batched_gemm_bf16", XQ, WQ, out, bias, int(splitK or 0))
    return out


@functools.lru_cache(maxsize=1024)
def compute_batched_gemm_SplitK(M: int, N: int, K: int, tile_m: int, tile_n: int, tile_k: int) -> int:
    """log2 of the K split that fills the machine (aiter/ops/batched_gemm_op_bf16.py:38-50), with this GPU's SM count."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count if torch.cuda.is_available() else 148
    tile_num = ((M + tile_m - 1) // tile_m) * ((N + tile_n - 1) // tile_n)
    per_tile = sms / tile_num
    splitK = 0
    while per_tile >= pow(2, splitK + 1) and (pow(2, splitK + 1) * tile_k) < 2 * K:
        splitK += 1
    return splitK


def get_CKBatchedGEMM_config(B: int, M: int, N: int, K: int):
    return _batched_table.lookup(M, N, K, B)


def batched_gemm_bf16_CK(XQ: Tensor, WQ: Tensor, bias: Tensor | None = None, dtype=dtypes.bf16, splitK: int | None = None) -> Tensor:
    assert dtype in [dtypes.bf16, dtypes.fp16], f"Output {dtype=} is currently not supported in batched_gemm_bf16"
    b, m, n, k = XQ.shape[0], XQ.shape[1], WQ.shape[1], XQ.shape[2]
    cfg = get_CKBatchedGEMM_config(b, m, n, k)
    Y = torch.empty(b, m, n, dtype=dtype, device=XQ.device)
    if cfg is not None and cfg.get("kernelId") not in (None, ""):
        # a tuned row names the tile and the K split; the plain entry point leaves both to the library
        return batched_gemm_bf16_tune(XQ, WQ, Y, int(cfg["kernelId"]), int(cfg.get("splitK") or 0) if splitK is None else splitK)
    return batched_gemm_bf16(XQ, WQ, Y, bias, 0 if splitK is None else splitK)


def batched_gemm_bf16_tune(XQ: Tensor, WQ: Tensor, out: Tensor, kernelId: int, splitK: int = 0) -> Tensor:
    """The same with the tile named by its id in the kernel menu (aiter_b200.kernel_list()) and log2 of the K split."""
    _ffi.call("batched_gemm_bf16_tune", XQ, WQ, out, int(kernelId), int(splitK))
    return out
