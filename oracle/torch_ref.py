"""Torch-on-CPU form of the GEMM oracle.  TEST / BASELINE INFRASTRUCTURE ONLY (never imported by the
product package).  Same arithmetic as oracle/mx_oracle.py, written with torch ops so that it uses every
host thread the way the reference's own torch path does (op_tests/test_gemm_a4w4.py:23-39,
op_tests/test_mxfp8fp4gemm.py:63-72): dequantise to fp32, torch.mm in fp32, cast to bf16.
Parity status: pinned through tests/test_oracle_golden.py (equal to the numpy oracle and to the
reference-generated golden outputs)."""
from __future__ import annotations

import torch

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def e8m0_to_f32(b: torch.Tensor) -> torch.Tensor:
    b = b.view(torch.uint8)
    bits = b.to(torch.int32) << 23
    bits = torch.where(b == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(b == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    return bits.view(torch.float32)


def dequant_fp8(bits: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    v = bits.view(torch.float8_e4m3fn).to(torch.float32)
    return v * e8m0_to_f32(scale[: v.shape[0]]).repeat_interleave(32, dim=1)[:, : v.shape[1]]


def dequant_fp4(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    b = packed.view(torch.uint8)
    nib = torch.stack((b & 0xF, b >> 4), dim=-1).flatten(-2).long()
    mag = torch.tensor(_E2M1, dtype=torch.float32)
    v = torch.cat((mag, -mag))[nib]
    return v * e8m0_to_f32(scale[: v.shape[0]]).repeat_interleave(32, dim=1)[:, : v.shape[1]]


def gemm_a8w8_mxfp8(a, b, sa, sb):
    return torch.mm(dequant_fp8(a, sa), dequant_fp8(b, sb).T).to(torch.bfloat16)


def gemm_a4w4(a, b, sa, sb):
    return torch.mm(dequant_fp4(a, sa), dequant_fp4(b, sb).T).to(torch.bfloat16)


def gemm_a8w4_mxfp8(a, b, sa, sb):
    return torch.mm(dequant_fp8(a, sa), dequant_fp4(b, sb).T).to(torch.bfloat16)


def gemm_a16w16(a, b, bias=None):
    return torch.nn.functional.linear(a.float(), b.float(), None if bias is None else bias.float()).to(torch.bfloat16)
