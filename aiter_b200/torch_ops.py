"""torch.library registration of the GEMM operators under the namespace `aiter`, with fake-tensor
implementations (output shape / dtype only), so that torch.compile, FakeTensorMode and meta-device
tracing see them as opaque ops -- the role of aiter/jit/utils/torch_guard.py:200-320 and of the
`gen_fake` functions next to each operator of the reference (e.g. gemm_a4w4_fake,
aiter/ops/gemm_op_a4w4.py:125-144).

    torch.ops.aiter.gemm_a4w4(A, B, A_scale, B_scale, bias, bpreshuffle)
    torch.ops.aiter.gemm_a8w8_mxfp8(A, B, ScaleA, ScaleB, a_preshuffle)
    torch.ops.aiter.gemm_a8w4_mxfp8(A, B, ScaleA, ScaleB, a_preshuffle)
    torch.ops.aiter.gemm_a8w8_blockscale(XQ, WQ, x_scale, w_scale, bpreshuffle)
    torch.ops.aiter.gemm_a16w16(A, B, bias)
    torch.ops.aiter.gemm_a4w4o4(A, B, A_scale, B_scale, apreshuffle, global_A_scale, global_B_scale)   packed fp4 [.., N/2]
    torch.ops.aiter.gemm_a4w4o8(A, B, A_scale, B_scale, apreshuffle, global_A_scale, global_B_scale)   (fp8 [.., N], e8m0 [.., N/128])
    torch.ops.aiter.gemm_nvfp4(A, B, ScaleA, ScaleB, global_A_scale, global_B_scale, a_preshuffle)
    torch.ops.aiter.batched_gemm_bf16(XQ, WQ)

The first five and the last two return a new bf16 tensor.  The real implementations call the operators of this package (CUDA only).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import batched_gemm_op_bf16, dtypes, gemm_op_a4w4, gemm_op_a8w4, gemm_op_a8w8, tuned_gemm

_NS = "aiter"


def _out(a: Tensor, n: int) -> Tensor:
    return a.new_empty((*a.shape[:-1], n), dtype=torch.bfloat16)


@torch.library.custom_op(f"{_NS}::gemm_a4w4", mutates_args=(), device_types="cuda")
def gemm_a4w4(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, bias: Optional[Tensor] = None,
              bpreshuffle: bool = True) -> Tensor:
    return gemm_op_a4w4.gemm_a4w4(A, B, A_scale, B_scale, bias=bias, bpreshuffle=bpreshuffle).clone()


@gemm_a4w4.register_fake
def _(A, B, A_scale, B_scale, bias=None, bpreshuffle=True):
    return _out(A, B.shape[0])


@torch.library.custom_op(f"{_NS}::gemm_a8w8_mxfp8", mutates_args=(), device_types="cuda")
def gemm_a8w8_mxfp8(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, a_preshuffle: bool = True) -> Tensor:
    return gemm_op_a8w8.gemm_a8w8_mxfp8(A, B, ScaleA, ScaleB, a_preshuffle=a_preshuffle)


@gemm_a8w8_mxfp8.register_fake
def _(A, B, ScaleA, ScaleB, a_preshuffle=True):
    return _out(A, B.shape[0])


@torch.library.custom_op(f"{_NS}::gemm_a8w4_mxfp8", mutates_args=(), device_types="cuda")
def gemm_a8w4_mxfp8(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, a_preshuffle: bool = True) -> Tensor:
    return gemm_op_a8w4.gemm_a8w4_mxfp8(A, B, ScaleA, ScaleB, a_preshuffle=a_preshuffle)


@gemm_a8w4_mxfp8.register_fake
def _(A, B, ScaleA, ScaleB, a_preshuffle=True):
    return _out(A, B.shape[0])


@torch.library.custom_op(f"{_NS}::gemm_a8w8_blockscale", mutates_args=(), device_types="cuda")
def gemm_a8w8_blockscale(XQ: Tensor, WQ: Tensor, x_scale: Tensor, w_scale: Tensor, bpreshuffle: bool = False) -> Tensor:
    return gemm_op_a8w8.gemm_a8w8_blockscale(XQ, WQ, x_scale, w_scale, isBpreshuffled=bpreshuffle)


@gemm_a8w8_blockscale.register_fake
def _(XQ, WQ, x_scale, w_scale, bpreshuffle=False):
    return _out(XQ, WQ.shape[0])


@torch.library.custom_op(f"{_NS}::gemm_a16w16", mutates_args=(), device_types="cuda")
def gemm_a16w16(A: Tensor, B: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    return tuned_gemm.gemm_a16w16(A, B, bias=bias)


@gemm_a16w16.register_fake
def _(A, B, bias=None):
    return _out(A, B.shape[0])


# low-precision outputs and NVFP4 inputs of the F4GEMM family (fake forms: aiter/ops/gemm_op_a4w4.py:463-474,519-534)
@torch.library.custom_op(f"{_NS}::gemm_a4w4o4", mutates_args=(), device_types="cuda")
def gemm_a4w4o4(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, apreshuffle: bool = False,
                global_A_scale: Optional[float] = None, global_B_scale: Optional[float] = None) -> Tensor:
    return gemm_op_a4w4.gemm_a4w4o4(A, B, A_scale, B_scale, apreshuffle=apreshuffle, global_A_scale=global_A_scale,
                                    global_B_scale=global_B_scale).view(torch.uint8)


@gemm_a4w4o4.register_fake
def _(A, B, A_scale, B_scale, apreshuffle=False, global_A_scale=None, global_B_scale=None):
    return A.new_empty((*A.shape[:-1], B.shape[0] // 2), dtype=torch.uint8)


@torch.library.custom_op(f"{_NS}::gemm_a4w4o8", mutates_args=(), device_types="cuda")
def gemm_a4w4o8(A: Tensor, B: Tensor, A_scale: Tensor, B_scale: Tensor, apreshuffle: bool = False,
                global_A_scale: Optional[float] = None, global_B_scale: Optional[float] = None) -> tuple[Tensor, Tensor]:
    o, sc = gemm_op_a4w4.gemm_a4w4o8(A, B, A_scale, B_scale, apreshuffle=apreshuffle, global_A_scale=global_A_scale,
                                     global_B_scale=global_B_scale)
    return o, sc.view(torch.uint8)


@gemm_a4w4o8.register_fake
def _(A, B, A_scale, B_scale, apreshuffle=False, global_A_scale=None, global_B_scale=None):
    n = B.shape[0]
    return (A.new_empty((*A.shape[:-1], n), dtype=dtypes.fp8),
            A.new_empty((*A.shape[:-1], n // gemm_op_a4w4.MXFP8_OUT_SCALE_BLOCK), dtype=torch.uint8))


@torch.library.custom_op(f"{_NS}::gemm_nvfp4", mutates_args=(), device_types="cuda")
def gemm_nvfp4(A: Tensor, B: Tensor, ScaleA: Tensor, ScaleB: Tensor, global_A_scale: float = 1.0, global_B_scale: float = 1.0,
               a_preshuffle: bool = True) -> Tensor:
    return gemm_op_a4w4.gemm_nvfp4_asm(A, B, ScaleA, ScaleB, global_A_scale, global_B_scale, a_preshuffle=a_preshuffle)


@gemm_nvfp4.register_fake
def _(A, B, ScaleA, ScaleB, global_A_scale=1.0, global_B_scale=1.0, a_preshuffle=True):
    return _out(A, B.shape[0])


@torch.library.custom_op(f"{_NS}::batched_gemm_bf16", mutates_args=(), device_types="cuda")
def batched_gemm_bf16(XQ: Tensor, WQ: Tensor) -> Tensor:
    return batched_gemm_op_bf16.batched_gemm_bf16_CK(XQ, WQ)


@batched_gemm_bf16.register_fake
def _(XQ, WQ):
    return XQ.new_empty((XQ.shape[0], XQ.shape[1], WQ.shape[1]), dtype=torch.bfloat16)
