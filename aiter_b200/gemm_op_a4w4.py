"""MXFP4 x MXFP4 GEMM entry points (reference: aiter/ops/gemm_op_a4w4.py:33-78,147-287,581-608)."""
from __future__ import annotations

import torch
from torch import Tensor

import logging

from . import _ffi, dtypes
from .config import TunedTable

logger = logging.getLogger("aiter")

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


# the mxfp8 output of the F4GEMM entry point carries one E8M0 scale per 128 output columns (gemm_op_a4w4.py:327-329)
MXFP8_OUT_SCALE_BLOCK = 128


def _alloc_f4gemm_out(M: int, N: int, dtype: torch.dtype, device) -> Tensor:
    """bf16 [M, N]; packed fp4 [M, N/2]; fp8 [M, N] (its scale is a separate tensor) (gemm_op_a4w4.py:337-346)."""
    if dtype == dtypes.fp4x2:
        assert N % 2 == 0, "packed fp4 output requires even N"
        return torch.empty((M, N // 2), dtype=torch.uint8, device=device).view(dtypes.fp4x2)
    return torch.empty((M, N), dtype=dtype, device=device)


def _alloc_f4gemm_out_scale(M: int, N: int, dtype: torch.dtype, device):
    """[M, N/128] e8m0 for the fp8 output, which the kernel fills in the packed (M/64, N/128, 16, 4) order; None
    otherwise (gemm_op_a4w4.py:349-362)."""
    if dtype != dtypes.fp8:
        return None
    assert N % MXFP8_OUT_SCALE_BLOCK == 0, f"mxfp8 output requires N % {MXFP8_OUT_SCALE_BLOCK} == 0, got N={N}"
    assert M % 64 == 0, f"mxfp8 output-scale packing requires M % 64 == 0, got M={M}"
    return torch.empty((M, N // MXFP8_OUT_SCALE_BLOCK), dtype=torch.uint8, device=device).view(dtypes.fp8_e8m0)


def unpack_mxfp8_out_scale(packed: Tensor, M: int, N: int) -> Tensor:
    """Packed (M/64, N/128, 16, 4) scale bytes -> row-major [M, N/128] (gemm_op_a4w4.py:365-380)."""
    assert M % 64 == 0, f"mxfp8 output-scale packing requires M % 64 == 0, got M={M}"
    assert N % MXFP8_OUT_SCALE_BLOCK == 0, f"mxfp8 output requires N % {MXFP8_OUT_SCALE_BLOCK} == 0, got N={N}"
    sn = N // MXFP8_OUT_SCALE_BLOCK
    u8 = packed.reshape(-1).view(torch.uint8)[: (M // 64) * sn * 64]
    return u8.reshape(M // 64, sn, 16, 4).permute(0, 3, 2, 1).reshape(M, sn).contiguous().view(dtypes.fp8_e8m0)


def gemm_mxfp4_asm(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, dtype: torch.dtype = dtypes.bf16,
                   a_preshuffle: bool = False, kernelName: str = ""):
    """MXFP4 GEMM with the (m/32,k/4,32,4) scale layout and 16x16-byte tiled operands (B always, A when a_preshuffle)
    (aiter/ops/gemm_op_a4w4.py:383-407).  dtype: bf16 [M,N]; fp4x2: packed e2m1 [M,N/2] of the unscaled product; fp8:
    (e4m3 [M,N], e8m0 scale per 128 columns in the packed (M/64,N/128,16,4) order - see unpack_mxfp8_out_scale)."""
    M, N = A.shape[0], B.shape[0]
    out = _alloc_f4gemm_out(M, N, dtype, A.device)
    out_scale = _alloc_f4gemm_out_scale(M, N, dtype, A.device)
    _ffi.call("mxfp4_gemm_asm", A, B, ScaleA, ScaleB, out, out_scale, kernelName if kernelName else None, int(bool(a_preshuffle)))
    return (out, out_scale) if out_scale is not None else out


def gemm_nvfp4_asm(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, GlobalScaleA: float, GlobalScaleB: float,
                   dtype: torch.dtype = dtypes.bf16, a_preshuffle: bool = True, kernelName: str = ""):
    """NVFP4 GEMM (aiter/ops/gemm_op_a4w4.py:410-443): D = gA * gB * (deq A)(deq B)^T with one e4m3 scale per 16
    elements, scales in tiles of 32 rows x 8 (shuffle_scale_f4(s, 8)), operands 16x16-byte tiled (B always, A when
    a_preshuffle).  dtype: bf16 [M,N]; fp4x2: packed e2m1 [M,N/2] of gA * gB * (raw product, block scales dropped);
    fp8: (e4m3 [M,N], e8m0 scale per 128 columns in the packed (M/64,N/128,16,4) order)."""
    M, N = A.shape[0], B.shape[0]
    out = _alloc_f4gemm_out(M, N, dtype, A.device)
    out_scale = _alloc_f4gemm_out_scale(M, N, dtype, A.device)
    _ffi.call("nvfp4_gemm_asm", A, B, ScaleA, ScaleB, float(GlobalScaleA), float(GlobalScaleB), out, out_scale,
              kernelName if kernelName else None, int(bool(a_preshuffle)))
    return (out, out_scale) if out_scale is not None else out


def _as_global_scale(scale) -> float:
    """An NVFP4 per-tensor scale given as a float or a one-element tensor -> float (gemm_op_a4w4.py:445-451)."""
    if scale is None:
        return 1.0
    if torch.is_tensor(scale):
        return float(scale.detach().reshape(-1)[0].item())
    return float(scale)


def _f4gemm_dispatch(A, B, A_scale, B_scale, *, dtype, apreshuffle, global_A_scale, global_B_scale, bias, alpha, beta):
    """The reference's gfx1250 F4GEMM dispatch (gemm_op_a4w4.py:80-122): bias / alpha / beta are not part of these
    kernels (a warning, as there); the presence of a per-tensor global scale selects NVFP4 over MXFP4."""
    if bias is not None or (alpha is not None and alpha != 1.0) or (beta is not None and beta != 0.0):
        logger.warning("the F4GEMM kernels ignore bias/alpha/beta.")
    m = A.numel() // A.shape[-1]
    A2 = A.view(m, A.shape[-1])
    if global_A_scale is not None or global_B_scale is not None:
        return gemm_nvfp4_asm(A2, B, A_scale, B_scale, _as_global_scale(global_A_scale), _as_global_scale(global_B_scale),
                              dtype=dtype, a_preshuffle=bool(apreshuffle))
    return gemm_mxfp4_asm(A2, B, A_scale, B_scale, dtype=dtype, a_preshuffle=bool(apreshuffle))


def gemm_a4w4o4(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, bias: Tensor | None = None, alpha: float | None = 1.0,
                beta: float | None = 0.0, bpreshuffle: bool | None = True, apreshuffle: bool | None = False,
                global_A_scale: Tensor | None = None, global_B_scale: Tensor | None = None) -> Tensor:
    """A4W4 GEMM with packed FP4 (e2m1) output [*lead, N/2] (gemm_op_a4w4.py:476-516).  As in the reference, whose
    fp4-output kernel is its "noscale" variant, the block scales are not applied: the fp32 product of the raw e2m1 values
    is cast to e2m1 (round to nearest even, saturating).  B 16x16-byte tiled, scales in the (m/32,k/4,32,4) order."""
    out = _f4gemm_dispatch(A, B, A_scale, B_scale, dtype=dtypes.fp4x2, apreshuffle=apreshuffle, global_A_scale=global_A_scale,
                           global_B_scale=global_B_scale, bias=bias, alpha=alpha, beta=beta)
    return out.view(*A.shape[:-1], out.shape[-1])


def gemm_a4w4o8(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, bias: Tensor | None = None, alpha: float | None = 1.0,
                beta: float | None = 0.0, bpreshuffle: bool | None = True, apreshuffle: bool | None = False,
                global_A_scale: Tensor | None = None, global_B_scale: Tensor | None = None):
    """A4W4 GEMM with mxfp8 output: (e4m3 data [*lead, N], E8M0 scale) with one RoundUp scale per 128 output columns,
    the scale in the packed (M/64, N/128, 16, 4) order - unpack with unpack_mxfp8_out_scale (gemm_op_a4w4.py:519-567)."""
    o, sc = _f4gemm_dispatch(A, B, A_scale, B_scale, dtype=dtypes.fp8, apreshuffle=apreshuffle, global_A_scale=global_A_scale,
                             global_B_scale=global_B_scale, bias=bias, alpha=alpha, beta=beta)
    lead = A.shape[:-1]
    return o.view(*lead, o.shape[-1]), sc.view(*lead, sc.shape[-1])


def gemm_a4w4(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, bias: Tensor | None = None,
              dtype: torch.dtype = dtypes.bf16, alpha: float | None = 1.0, beta: float | None = 0.0,
              bpreshuffle: bool | None = True, apreshuffle: bool | None = False,
              global_A_scale: Tensor | None = None, global_B_scale: Tensor | None = None) -> Tensor:
    """A4W4 GEMM returning one bf16 tensor [.., N].  The tuned table chooses the kernel and split-K for
    (M, N, K); untuned shapes use the library heuristic."""
    if dtype in (dtypes.fp4x2, dtypes.fp8):
        raise NotImplementedError("gemm_a4w4 returns one plain-dtype tensor; use gemm_a4w4o4 / gemm_a4w4o8")
    if global_A_scale is not None or global_B_scale is not None:
        # NVFP4 inputs come in the F4GEMM wire formats (16x16-byte tiled B, scales in tiles of 32 rows x 8), as on the
        # reference's F4GEMM architecture (gemm_op_a4w4.py:178-193)
        out = _f4gemm_dispatch(A, B, A_scale, B_scale, dtype=dtype, apreshuffle=bool(apreshuffle), global_A_scale=global_A_scale,
                               global_B_scale=global_B_scale, bias=bias, alpha=alpha, beta=beta)
        return out.view(*A.shape[:-1], out.shape[-1])
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
