"""Operand and scale layout permutations (bit-identical to the reference's aiter/ops/shuffle.py).

On B200 these layouts are consumed as they are: a (16,16)-shuffled weight is a sequence of
16-row x 16-byte tiles, i.e. pairs of 8x16-byte tensor-core core matrices, which TMA drops
into shared memory as an un-swizzled K-major operand; the scale layouts are re-ordered inside
the GEMM kernel.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


def _as_bytes(x: Tensor):
    if hasattr(torch, "float4_e2m1fn_x2") and x.dtype == torch.float4_e2m1fn_x2:
        return x.view(torch.uint8)
    return x


def _retile(src: Tensor, rows_per_tile: int, cols_per_tile: int) -> Tensor:
    """[R, C] -> tiles of (rows_per_tile x cols_per_tile), tile-row-major, rows outer in a tile."""
    r, c = src.shape
    assert r % rows_per_tile == 0, f"rows={r} must be divisible by {rows_per_tile}"
    assert c % cols_per_tile == 0, f"cols={c} must be divisible by {cols_per_tile}"
    t = src.reshape(r // rows_per_tile, rows_per_tile, c // cols_per_tile, cols_per_tile)
    return t.transpose(1, 2).contiguous().view(r, c)


def shuffle_weight(x: Tensor, layout=(16, 16), use_int4=False, is_guinterleave=False, gate_up: bool = False,
                   pad_k_to: int = 0) -> Tensor:
    """[.., N, K] -> [.., N/16][K bytes/32][2][16 rows][16 bytes] (shuffle.py:148-209).
    The result carries `.is_shuffled = True`, which gemm_a16w16 reads."""
    if use_int4 or is_guinterleave:
        raise NotImplementedError("int4 / gate-up interleaved weight shuffles belong to the MoE path, which is not built")
    x_type = x.dtype
    x = _as_bytes(x)
    original_k = x.shape[-1]
    if pad_k_to:
        if pad_k_to < 0:
            raise ValueError(f"pad_k_to must be non-negative, got {pad_k_to}")
        padded_k = -(-original_k // pad_k_to) * pad_k_to
        if padded_k != original_k:
            x = F.pad(x.contiguous(), (0, padded_k - original_k), value=0)
    rows_in, bytes_in = layout
    vec = 16 // x.element_size()  # elements per 16-byte vector
    k_tile = bytes_in * 2
    assert x.shape[-2] % rows_in == 0, f"{x.shape[-2]} % {rows_in} == {x.shape[-2] % rows_in}"
    assert x.shape[-1] % k_tile == 0, f"{x.shape[-1]} % {k_tile} == {x.shape[-1] % k_tile}"
    t = x.reshape(-1, x.shape[-2] // rows_in, rows_in, x.shape[-1] // k_tile, k_tile // vec, vec)
    out = t.permute(0, 1, 3, 4, 2, 5).contiguous().view(*x.shape).view(x_type)
    out.is_shuffled = True
    if pad_k_to:
        out.aiter_original_k = original_k
        out.aiter_padded_k = x.shape[-1]
    return out


def shuffle_scale(src: Tensor, experts_cnt=None, is_guinterleave: bool = False, gate_up: bool = False) -> Tensor:
    """E8M0 scales [M, K/32] -> padded to (256, 8) multiples and stored so that byte
    (m, k) sits at (m/32*sn)*32 + (k/8)*256 + (k%4)*64 + (m%16)*4 + ((k%8)/4)*2 + (m%32)/16
    (shuffle.py:339-365).  Padding bytes are set to 0x7F (scale 1.0); the reference leaves them
    uninitialised."""
    if src is None or src.dtype == torch.float32:
        return src
    if is_guinterleave:
        raise NotImplementedError("gate-up interleaved scale shuffle belongs to the MoE path, which is not built")
    assert src.ndim == 2, "scale must be a 2D tensor"
    m, n = src.shape
    sm, sn = -(-m // 256) * 256, -(-n // 8) * 8
    padded = torch.full((sm, sn), 0x7F, dtype=torch.uint8, device=src.device)
    padded[:m, :n] = src.view(torch.uint8)
    t = padded.view(sm // 32, 2, 16, sn // 8, 2, 4).permute(0, 3, 5, 2, 4, 1).contiguous()
    return t.view(sm, sn).view(src.dtype)


def shuffle_mxfp8fp4_a(src: Tensor) -> Tensor:
    """Activation tiling (m, k) -> (m/2, k/128, 2, 128) over bytes (shuffle.py:29-41)."""
    return _retile(src.view(torch.uint8), 2, 128).view(src.dtype)


def shuffle_mxfp8fp4_b(src: Tensor) -> Tensor:
    """Weight 16x16-byte tile transpose (shuffle.py:44-57); identical to shuffle_weight(layout=(16,16))
    for one-byte elements."""
    return _retile(_as_bytes(src).view(torch.uint8), 16, 16).view(src.dtype)


def shuffle_mxfp8fp4_scale(src: Tensor) -> Tensor:
    """E8M0 scales: rows padded to 32 with 0x7F, then (m, k) -> (m/32, k/4, 32, 4) (shuffle.py:58-76)."""
    s = src.view(torch.uint8)
    pad = (-s.shape[0]) % 32
    if pad:
        s = F.pad(s, (0, 0, 0, pad), value=0x7F)
    return _retile(s, 32, 4).view(src.dtype)


def shuffle_weight_f4(src: Tensor) -> Tensor:
    """Packed-fp4 operand [rows, K/2] -> 16x16-byte tile transpose (shuffle.py:319-336); the layout the F4GEMM entry
    point takes for B, and for A when a_preshuffle is set."""
    return _retile(_as_bytes(src).view(torch.uint8), 16, 16).view(src.dtype)


def shuffle_scale_f4(src: Tensor, intype: int = 7) -> Tensor:
    """F4GEMM scale pre-shuffle (shuffle.py:293-316): [M, K/block] -> tiles of 32 rows x 4 (MXFP4, intype 7) or
    32 rows x 8 (NVFP4, intype 8) scale columns, rows outer inside a tile.  No row padding: M % 32 == 0."""
    return _retile(src.view(torch.uint8), 32, 8 if intype == 8 else 4).view(src.dtype)
