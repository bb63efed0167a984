"""dtype aliases and the AiterDtype numbering (reference: aiter/utility/dtypes.py:26-60,
csrc/include/aiter_enum.h:34-50)."""
import enum

import torch

_8bit_fallback = torch.uint8
i4x2 = getattr(torch, "int4", _8bit_fallback)
fp4x2 = getattr(torch, "float4_e2m1fn_x2", _8bit_fallback)
fp8 = torch.float8_e4m3fn
fp8_e8m0 = getattr(torch, "float8_e8m0fnu", _8bit_fallback)
fp16 = torch.float16
bf16 = torch.bfloat16
fp32 = torch.float32
u32 = torch.uint32
i32 = torch.int32
i16 = torch.int16
i8 = torch.int8
u8 = torch.uint8
i64 = torch.int64
u64 = torch.uint64

aiter_dtypes = {
    "fp8": 0, "fp8_e8m0": 1, "fp16": 2, "bf16": 3, "fp32": 4, "i4x2": 5, "fp4x2": 6,
    "u32": 7, "i32": 8, "i16": 9, "i8": 10, "u8": 11, "i64": 12, "u64": 13,
}
d_dtypes = {name: globals()[name] for name in aiter_dtypes}
globals().update({f"AITER_DTYPE_{name}": idx for name, idx in aiter_dtypes.items()})
# later names win on purpose: when an alias falls back to uint8 the id must be "u8"
_torch_to_aiter_dtype = {}
for _name in ("i4x2", "fp4x2", "fp8_e8m0", "fp8", "fp16", "bf16", "fp32", "u32", "i32", "i16", "i8", "u8", "i64", "u64"):
    _torch_to_aiter_dtype[globals()[_name]] = aiter_dtypes[_name]


def aiter_dtype_id(dtype) -> int:
    try:
        return _torch_to_aiter_dtype[dtype]
    except KeyError:
        raise AssertionError(f"Unsupported dtype: {dtype}") from None


class QuantType(enum.IntEnum):
    """csrc/include/aiter_enum.h:16-26."""
    No = 0
    per_Tensor = 1
    per_Token = 2
    per_1x32 = 3
    per_1x128 = 4
    per_128x128 = 5
    per_256x128 = 6
    per_1024x128 = 7


class MxScaleRoundMode(enum.IntEnum):
    """aiter/utility/mx_types.py:36-48."""
    RoundDown = 0
    RoundUp = 1
    Even = 2
    Ceil = 3


class MxDtype(enum.IntEnum):
    """aiter/utility/mx_types.py:51-56."""
    FP4_E2M1 = 0
    FP8_E4M3 = 1
    FP8_E4M3_FNUZ = 2


MX_DEFAULT_ROUND_MODE = MxScaleRoundMode.RoundUp


def str2tuple(v):
    return tuple(int(p) for p in str(v).strip("()").split(",") if p.strip())
