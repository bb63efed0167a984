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


def get_torch_quant(qType):
    table = {
        QuantType.No: lambda *a, **k: (a[0], None),
        QuantType.per_1x32: per_1x32_f4_quant,
    }

    def unsupported(*a, **k):
        raise NotImplementedError(f"unsupported quant type {qType=}")

    return table.get(QuantType(int(qType)), unsupported)
