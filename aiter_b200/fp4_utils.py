"""MX numerics on torch tensors (any device): E8M0 block scales, E2M1 / E4M3 element codes.

Same results, bit for bit, as the reference's torch path (aiter/utility/fp4_utils.py); the
algorithms are restated, not transcribed: E2M1 rounding is a count of crossed rounding
thresholds instead of mantissa bit arithmetic.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import dtypes
from .dtypes import MX_DEFAULT_ROUND_MODE, MxDtype, MxScaleRoundMode

_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# (target_max_pow2, max_pos, mantissa bits) per element type - fp4_utils.py:77-81
_DTYPE_CFG = {
    int(MxDtype.FP4_E2M1): (2, 6.0, 1),
    int(MxDtype.FP8_E4M3): (8, 448.0, 3),
    int(MxDtype.FP8_E4M3_FNUZ): (7, 240.0, 3),
}


def _exponent_floor(x: Tensor) -> Tensor:
    bits = x.contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF).to(torch.uint8)


def _exponent_ceil(x: Tensor) -> Tensor:
    bits = x.contiguous().view(torch.int32)
    exp = (bits >> 23) & 0xFF
    bump = ((bits & 0x7FFFFF) != 0) & (exp < 0xFF)
    return (exp + bump.to(torch.int32)).to(torch.uint8)


def f32_to_mx_e8m0_scale(amax: Tensor, *, mode: int = MX_DEFAULT_ROUND_MODE, dtype: int = MxDtype.FP4_E2M1) -> Tensor:
    """Per-block E8M0 scale byte from the block's max |x| (fp4_utils.py:85-158).

    RoundUp (default): ceil_pow2(amax / max_pos) with a true fp32 division."""
    mode, dtype = int(mode), int(dtype)
    if dtype not in _DTYPE_CFG:
        raise ValueError(f"f32_to_mx_e8m0_scale: unsupported dtype {dtype!r}; supported: {list(_DTYPE_CFG)}")
    pow2, max_pos, mbits = _DTYPE_CFG[dtype]
    amax = amax.to(torch.float32)
    if mode == MxScaleRoundMode.RoundUp:
        out = _exponent_ceil(amax / max_pos)
    elif mode == MxScaleRoundMode.RoundDown:
        out = _exponent_floor(amax / float(1 << pow2))
    elif mode == MxScaleRoundMode.Ceil:
        out = _exponent_ceil(amax / float(1 << pow2))
    elif mode == MxScaleRoundMode.Even:
        bits = amax.contiguous().view(torch.int32)
        rounded = ((bits + (1 << (23 - mbits - 1))) & -0x800000).view(torch.float32)
        out = _exponent_floor(rounded / float(1 << pow2))
    else:
        raise ValueError(f"f32_to_mx_e8m0_scale: unknown mode {mode!r} (expected 0=RoundDown, 1=RoundUp, 2=Even, 3=Ceil)")
    return out.view(dtypes.fp8_e8m0)


def fp4_f32_to_e8m0_scale(amax: Tensor) -> Tensor:
    return f32_to_mx_e8m0_scale(amax, mode=MX_DEFAULT_ROUND_MODE, dtype=MxDtype.FP4_E2M1)


def e8m0_to_f32(scale: Tensor) -> Tensor:
    """2^(byte-127); byte 0 -> 2^-127, byte 255 -> NaN (fp4_utils.py:213-221)."""
    b = scale.view(torch.uint8)
    bits = b.to(torch.int32) << 23
    bits = torch.where(b == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(b == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    return bits.view(torch.float32)


def f32_to_e2m1_code(x: Tensor) -> Tensor:
    """fp32 -> E2M1 code in the low nibble of a uint8: round to nearest, ties to the even code,
    saturate at +-6, keep the sign bit of zero (fp4_utils.py:255-370)."""
    x = x.to(torch.float32)
    a = x.abs()
    code = (
        (a > 0.25).to(torch.uint8)
        + (a >= 0.75).to(torch.uint8)
        + (a > 1.25).to(torch.uint8)
        + (a >= 1.75).to(torch.uint8)
        + (a > 2.5).to(torch.uint8)
        + (a >= 3.5).to(torch.uint8)
        + (a > 5.0).to(torch.uint8)
    )
    sign = ((x.contiguous().view(torch.int32) >> 28) & 0x8).to(torch.uint8)
    return code | sign


def pack_uint4(codes: Tensor) -> Tensor:
    """Even index -> low nibble (fp4_utils.py:235-240)."""
    assert codes.shape[-1] % 2 == 0, f"{tuple(codes.shape)} last dim not divisible by two"
    c = codes.contiguous()
    return c[..., 0::2] | (c[..., 1::2] << 4)


def f32_to_mxfp4(x: Tensor) -> Tensor:
    return pack_uint4(f32_to_e2m1_code(x)).view(dtypes.fp4x2)


def mxfp4_to_f32(x: Tensor) -> Tensor:
    """Packed E2M1 -> fp32, twice as many elements along the last dim (fp4_utils.py:25-52)."""
    b = x.view(torch.uint8)
    nib = torch.stack((b & 0xF, b >> 4), dim=-1).flatten(-2)
    mag = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=b.device)
    lut = torch.cat((mag, -mag))
    return lut[nib.long()]


def e8m0_shuffle(scale: Tensor) -> Tensor:
    from .shuffle import shuffle_scale

    return shuffle_scale(scale)
