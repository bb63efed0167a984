"""Block quantisers of the GEMM inputs (reference torch path: aiter/ops/quant.py:97-204,272-315)."""
from __future__ import annotations

import torch
from torch import Tensor

from . import dtypes, fp4_utils
from .dtypes import MX_DEFAULT_ROUND_MODE, MxDtype, QuantType


def _block_amax(x: Tensor, block: int):
    flat = x.reshape(-1, block)
    return flat, flat.float().abs().amax(dim=1)


def per_1x32_f4_quant(x: Tensor, scale=None, quant_dtype=dtypes.fp4x2, shuffle: bool = False, pack_dim: int = -1,
                      round_mode=MX_DEFAULT_ROUND_MODE):
    """[.., K] -> (packed E2M1 [.., K/2], E8M0 scales [M, K/32]); scale = RoundUp(amax / 6) by default,
    elements RNE with saturation.  `shuffle=True` stores the scales in the e8m0_shuffle layout.
    pack_dim=0 quantises a [K, N] right-hand side along its first dim."""
    assert quant_dtype == dtypes.fp4x2
    transposed = False
    if pack_dim == 0:
        assert x.dim() == 2, "pack_dim=0 requires a 2D input tensor (K, N)"
        x, transposed = x.T.contiguous(), True
    shape = x.shape
    rows = x.numel() // shape[-1]
    blocks, amax = _block_amax(x, 32)
    try:
        sb = fp4_utils.f32_to_mx_e8m0_scale(amax, mode=round_mode, dtype=MxDtype.FP4_E2M1)
    except ValueError as e:
        raise ValueError(
            f"per_1x32_f4_quant: invalid round_mode={round_mode!r} (type={type(round_mode).__name__}); "
            "expected 0 (RoundDown/FLOOR), 1 (RoundUp/RCEIL), 2 (Even), 3 (Ceil), or any MxScaleRoundMode value."
        ) from e
    y = fp4_utils.f32_to_mxfp4(blocks.float() / fp4_utils.e8m0_to_f32(sb).view(-1, 1)).view(*shape[:-1], -1)
    sb = sb.view(torch.uint8).view(rows, -1)
    if shuffle:
        sb = fp4_utils.e8m0_shuffle(sb)
    sb = sb.view(dtypes.fp8_e8m0)
    if transposed:
        y = y.T.contiguous()
        sb = sb.view(torch.uint8).T.contiguous().view(dtypes.fp8_e8m0)
    return y, sb


def per_1x32_f8_scale_f8_quant(x: Tensor, scale=None, quant_dtype=dtypes.fp8, scale_type=dtypes.fp32, shuffle: bool = False):
    """[.., K] -> (e4m3 [.., K], per-32 scales [M, K/32]); scale_type fp8_e8m0 gives RoundUp(amax / 448) bytes,
    fp32 gives amax / 256 (quant.py:272-315)."""
    assert quant_dtype == dtypes.fp8
    shape = x.shape
    rows = x.numel() // shape[-1]
    blocks, amax = _block_amax(x, 32)
    if scale_type == dtypes.fp32:
        sf = amax / 256.0  # 2^floor(log2(448))
        sb = None
    else:
        sb = fp4_utils.f32_to_mx_e8m0_scale(amax, mode=MX_DEFAULT_ROUND_MODE, dtype=MxDtype.FP8_E4M3)
        sf = fp4_utils.e8m0_to_f32(sb)
    y = (blocks.float() / sf.view(-1, 1)).view(shape).to(quant_dtype)
    if sb is None:
        return y, sf.view(rows, -1)
    sb = sb.view(rows, -1)
    if shuffle:
        sb = fp4_utils.e8m0_shuffle(sb)
    return y, sb


def dynamic_per_group_scaled_quant(out: Tensor, input: Tensor, scales: Tensor, group_size: int = 32, shuffle_scale=True,
                                   num_rows: Tensor | None = None, num_rows_factor: int = 1) -> None:
    """CUDA 1x32 MX quantiser (aiter/ops/quant.py:766-791): `out.dtype` selects MXFP4 (fp4x2 / uint8) or MXFP8 (fp8);
    `scales` receives e8m0 bytes.  shuffle_scale: False plain [M, K/32]; True e8m0_shuffle order; 2 the
    (m/32, k/4, 32, 4) order the MXFP8 GEMM entry points take."""
    from . import _ffi

    _ffi.call("dynamic_per_group_scaled_quant", out, input, scales, group_size, int(shuffle_scale), num_rows, num_rows_factor)


def per_1x32_mx_quant_hip(x: Tensor, scale=None, quant_dtype=dtypes.fp4x2, shuffle=False, num_rows: Tensor | None = None,
                          num_rows_factor: int = 1, scale_type=None):
    """Fused dynamic 1x32 MX quantisation on the GPU (aiter/ops/quant.py:486-597): returns (y, scale) with the scales
    already in the layout the GEMM reads.  fp4x2: y [M, K/2], e8m0 scales [M, K/32], or [pad256(M), pad8(K/32)] in
    e8m0_shuffle order when shuffle=True.  fp8 (scale_type must be fp8_e8m0 here): y [M, K] e4m3, same scale shapes;
    shuffle=2 gives the (m/32, k/4, 32, 4) order of the MXFP8 GEMMs in a [pad32(M), K/32] array."""
    if scale is not None:
        raise ValueError("unsupported: static per token quant")
    assert x.dim() == 2, "per_1x32_mx_quant_hip takes a 2-D input"
    m, n = x.shape
    assert n % 32 == 0, f"n={n} must be divisible by 32"
    if quant_dtype == dtypes.fp4x2:
        if scale_type is not None and scale_type != dtypes.fp8_e8m0:
            raise ValueError(f"per_1x32_mx_quant_hip: fp4x2 output requires e8m0 scale; got scale_type={scale_type}")
        out_cols = n // 2
    elif quant_dtype == dtypes.fp8:
        if scale_type is None or scale_type == dtypes.fp32:
            raise NotImplementedError("per_1x32_mx_quant_hip(fp8): only scale_type=dtypes.fp8_e8m0 runs on the GPU here; "
                                      "fp32 scales: per_1x32_f8_scale_f8_quant")
        if scale_type != dtypes.fp8_e8m0:
            raise ValueError(f"per_1x32_mx_quant_hip: fp8 output expects scale_type in {{fp32, fp8_e8m0}}, got {scale_type}")
        out_cols = n
    else:
        raise ValueError(f"per_1x32_mx_quant_hip: unsupported quant_dtype {quant_dtype}, expected one of (dtypes.fp4x2, dtypes.fp8)")
    kb = n // 32
    if shuffle == 2:
        shape = ((m + 31) // 32 * 32, kb)
    elif shuffle:
        shape = ((m + 255) // 256 * 256, (kb + 7) // 8 * 8)
    else:
        shape = (m, kb)
    scale = torch.empty(shape, dtype=torch.uint8, device=x.device).view(dtypes.fp8_e8m0)
    y = torch.empty((m, out_cols), dtype=torch.uint8, device=x.device).view(quant_dtype)
    dynamic_per_group_scaled_quant(y, x, scale, 32, shuffle_scale=shuffle, num_rows=num_rows, num_rows_factor=num_rows_factor)
    return y, scale


def per_1x32_f4_quant_hip(x: Tensor, scale=None, quant_dtype=dtypes.fp4x2, shuffle=False, num_rows: Tensor | None = None,
                          num_rows_factor: int = 1):
    """fp4-only wrapper kept for callers of the older name (aiter/ops/quant.py:600-626)."""
    assert quant_dtype == dtypes.fp4x2, "per_1x32_f4_quant_hip is fp4-only; use per_1x32_mx_quant_hip for fp8"
    return per_1x32_mx_quant_hip(x, scale=scale, quant_dtype=quant_dtype, shuffle=shuffle, num_rows=num_rows,
                                 num_rows_factor=num_rows_factor)


def get_hip_quant(qType):
    """QuantType.per_1x32 -> the fused GPU quantiser; other quant types are outside this library's path."""
    from .dtypes import QuantType

    if qType == QuantType.per_1x32:
        return per_1x32_mx_quant_hip
    raise NotImplementedError(f"get_hip_quant({qType}): only QuantType.per_1x32 is built")


def get_torch_quant(qType):
    table = {
        QuantType.No: lambda *a, **k: (a[0], None),
        QuantType.per_1x32: per_1x32_f4_quant,
    }

    def unsupported(*a, **k):
        raise NotImplementedError(f"unsupported quant type {qType=}")

    return table.get(QuantType(int(qType)), unsupported)
