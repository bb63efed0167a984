"""MXFP8 x MXFP8 GEMM (reference: aiter/ops/gemm_op_a8w8.py:1215-1254) with table-driven dispatch."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _ffi, dtypes, fp4_utils
from .config import TunedTable, get_cu_num

_mxfp8_table = TunedTable("a8w8_mxfp8")
_blockscale_table = TunedTable("a8w8_blockscale")
_blockscale_bpreshuffle_table = TunedTable("a8w8_blockscale_bpreshuffle")


def get_CKGEMM_config(M: int, N: int, K: int, bpreshuffle: bool = False):
    """Tuned row of the fp32-blockscale tables for (M, N, K), or None (reference: gemm_op_a8w8.py:441-483)."""
    return (_blockscale_bpreshuffle_table if bpreshuffle else _blockscale_table).lookup(M, N, K)


def _mxfp8_kernel_for(m: int, n: int, k: int) -> str:
    """e8m0-scaled blockscale problems run on the MXFP8 kernels: their tuned table names the configuration.
    For few rows no name is passed on: the library's few-rows blockscale kernel reads the e8m0 bytes itself."""
    if m <= 64:
        return ""
    # 65..256 rows: the same kernel on tiles of 64 rows while all of them fit the machine at once (the launcher's rule)
    if m <= 256 and k <= 32768 and -(-n // 128) * -(-m // 64) <= get_cu_num():
        return ""
    row = _mxfp8_table.lookup(m, n, k)
    return str(row.get("kernelName") or "") if row is not None else ""


def _is_e8m0(s: Tensor) -> bool:
    return s.dtype in (dtypes.fp8_e8m0, torch.uint8)


def _blockscale_scales(x_scale: Tensor, w_scale: Tensor):
    """Both e8m0: passed on as bytes (powers of two ride the block-scaled MMA: the problem runs on the MXFP8 kernel).
    Otherwise both go to fp32, e8m0 ones widened first as the reference does (gemm_op_a8w8.py:952-956)."""
    if _is_e8m0(x_scale) and _is_e8m0(w_scale):
        return x_scale, w_scale
    return (fp4_utils.e8m0_to_f32(x_scale) if _is_e8m0(x_scale) else x_scale,
            fp4_utils.e8m0_to_f32(w_scale) if _is_e8m0(w_scale) else w_scale)


def _blockscale_choice(cfg, scales_are_e8m0: bool, m: int, n: int, k: int):
    """-> (splitK, kernelName) for the library call.  The blockscale tables are tuned with fp32 scales: their
    bs_128x128 / bs_256x256 rows do not apply to e8m0-scaled problems, which run on the few-rows kernel (a
    bs_fewrows row stays valid: that kernel reads either scale type) or on the MXFP8 kernel its own table names."""
    splitK, kernelName = (int(cfg.get("splitK") or 0), str(cfg.get("kernelName") or "")) if cfg is not None else (0, "")
    if scales_are_e8m0 and not kernelName.startswith("bs_fewrows"):
        splitK, kernelName = 0, _mxfp8_kernel_for(m, n, k)
    return splitK, kernelName


def gemm_a8w8_blockscale(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, dtype: torch.dtype = dtypes.bf16,
                         isBpreshuffled: bool = False) -> Tensor:
    """Y[M,N] = (XQ * x_scale) @ (WQ * w_scale)^T with fp32 scales per 128-wide K block: x_scale [M, K/128],
    w_scale [ceil(N/128), K/128]; WQ row-major [N, K] (reference: gemm_op_a8w8.py:797-865)."""
    assert dtype in (dtypes.bf16, dtypes.fp16), f"Output {dtype=} is currently not supported in gemm_a8w8"
    if isBpreshuffled:
        return gemm_a8w8_blockscale_bpreshuffle(XQ, WQ, x_scale, w_scale, dtype)
    m, n, k = XQ.shape[0], WQ.shape[0], XQ.shape[1]
    Y = torch.empty(m, n, dtype=dtype, device=XQ.device)
    xs, ws = _blockscale_scales(x_scale, w_scale)
    splitK, kernelName = _blockscale_choice(get_CKGEMM_config(m, n, k), _is_e8m0(xs), m, n, k)
    _ffi.call("gemm_a8w8_blockscale", XQ, WQ, xs, ws, Y, splitK, kernelName or None)
    return Y


def gemm_a8w8_blockscale_bpreshuffle(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor,
                                     dtype: torch.dtype = dtypes.bf16) -> Tensor:
    """Same math with WQ (16,16)-shuffled and x_scale stored K-block-major ([K/128][M] in memory, passed either
    as the transposed-strided [M, K/128] view or re-viewed as a contiguous [M, K/128]); e8m0 scales are widened
    to fp32 first (reference: gemm_op_a8w8.py:895-1055)."""
    assert dtype in (dtypes.bf16, dtypes.fp16), f"Output {dtype=} is currently not supported in gemm_a8w8"
    m, n, k = XQ.shape[0], WQ.shape[0], XQ.shape[1]
    Y = torch.empty(m, n, dtype=dtype, device=XQ.device)
    xs, ws = _blockscale_scales(x_scale, w_scale)
    splitK, kernelName = _blockscale_choice(get_CKGEMM_config(m, n, k, bpreshuffle=True), _is_e8m0(xs), m, n, k)
    _ffi.call("gemm_a8w8_blockscale_bpreshuffle", XQ, WQ, xs, ws, Y, splitK, kernelName or None)
    return Y


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


def gemm_a8w8_blockscale_cktile(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, Out: Tensor, preshuffleB: bool = False,
                                splitK: int = 0, kernelName: str = "") -> Tensor:
    """The CK-tile back-end's name and argument order (csrc/include/rocm_ops.hpp:749-759); same kernels as gemm_a8w8_blockscale."""
    xs, ws = _blockscale_scales(x_scale, w_scale)
    _ffi.call("gemm_a8w8_blockscale_cktile", XQ, WQ, xs, ws, Out, int(bool(preshuffleB)), splitK, kernelName or None)
    return Out


def gemm_a8w8_blockscale_bpreshuffle_cktile(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, Out: Tensor,
                                            preshuffleB: bool = True, kernelName: str = "") -> Tensor:
    xs, ws = _blockscale_scales(x_scale, w_scale)
    _ffi.call("gemm_a8w8_blockscale_bpreshuffle_cktile", XQ, WQ, xs, ws, Out, int(bool(preshuffleB)), kernelName or None)
    return Out


def flatmm_a8w8_blockscale_asm(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, out: Tensor) -> Tensor:
    """aiter/ops/gemm_op_a8w8.py:342-362: row-major weight, fp32 scales, caller-provided output."""
    _ffi.call("flatmm_a8w8_blockscale_asm", XQ, WQ, x_scale, w_scale, out)
    return out


def gemm_a8w8_blockscale_bpreshuffle_asm(A: Tensor, B: Tensor, out: Tensor, A_scale: Tensor, B_scale: Tensor, bias: Tensor | None = None,
                                         splitK: int | None = None, kernelName: str | None = None, bpreshuffle: bool | None = True,
                                         zero_bias_buf: Tensor | None = None) -> Tensor:
    """aiter/ops/gemm_op_a8w8.py:397-423 (the assembly back-end's argument order; A_scale K-block-major as in
    gemm_a8w8_blockscale_bpreshuffle)."""
    _ffi.call("gemm_a8w8_blockscale_bpreshuffle_asm", A, B, out, A_scale, B_scale, bias, splitK if splitK is not None else -1, kernelName,
              int(bpreshuffle) if bpreshuffle is not None else 1, zero_bias_buf)
    return out
