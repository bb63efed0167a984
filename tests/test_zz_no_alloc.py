"""The allocation-free MXFP8 GEMM entry point against the regular one (collected last on purpose).

Some callers may not allocate device memory at all: a server that handed every byte to one arena at
start-up, a plugin living inside a host process whose allocator it must leave alone, a loop where a
driver allocation (which may synchronise the device) is not acceptable.  For them the library offers
aiter_b200_gemm_a8w8_mxfp8_noalloc: same arguments and results as mxfp8_mxfp8_gemm_asm, but its split-K
scratch is a fixed array inside the library image.  The test drives it through the C ABI twice in a row
(the array keeps the first call's contents, so the second call proves nothing stale leaks through) and
compares both results with the regular entry point and with the oracle.
"""
import pytest
import torch

from oracle import mx_oracle as ox
from tests.helpers import check, quant_fp8, randn_bf16, to_cuda_u8

pytestmark = pytest.mark.gpu


def _problem(ab, M, N, K, seed):
    x, w = randn_bf16(M, K, seed + 1), randn_bf16(N, K, seed + 2)
    xq, xs = quant_fp8(x)
    wq, ws = quant_fp8(w)
    ref = ox.gemm_a8w8_mxfp8_ref(xq, wq, xs, ws)
    args = (to_cuda_u8(xq, torch.float8_e4m3fn), ab.shuffle_mxfp8fp4_b(to_cuda_u8(wq, torch.float8_e4m3fn)),
            ab.shuffle_mxfp8fp4_scale(to_cuda_u8(xs)), ab.shuffle_mxfp8fp4_scale(to_cuda_u8(ws)))
    return ref, args


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    import aiter_b200 as ab
    from aiter_b200 import _ffi

    for (M, N, K, l2) in ((16, 512, 4096, 2), (200, 768, 1024, 1)):
        ref, (A, B, sA, sB) = _problem(ab, M, N, K, seed=40 + M)
        want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        _ffi.call("mxfp8_mxfp8_gemm_asm", A, B, sA, sB, want, None, 0)
        check(ref, want, what=f"regular entry point {M}x{N}x{K}")
        for attempt in (1, 2):
            got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            _ffi.call("aiter_b200_gemm_a8w8_mxfp8_noalloc", A, B, sA, sB, got, 0, l2)
            check(ref, got, what=f"no-alloc entry point, call {attempt}, {M}x{N}x{K} split 2^{l2}")
            diff = (got.float() - want.float()).abs()
            tol = 1e-2 + 1e-2 * want.float().abs()
            assert bool((diff <= tol).all()), f"call {attempt}: differs from the regular entry point by up to {diff.max().item()}"
            # this entry point keeps its own status record inside the fixed array: read that one, through the C ABI
            assert ab.noalloc_status(0) == (0, 0, 0, 0)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_noalloc_entry_point_refuses_what_does_not_fit():
    import aiter_b200 as ab

    # 8192 x 4096 output with a 16-way K split would need far more than 8 MiB of partial sums
    M, N, K = 8192, 4096, 2048
    A = torch.zeros((M, K), dtype=torch.float8_e4m3fn, device="cuda")
    B = torch.zeros((N, K), dtype=torch.float8_e4m3fn, device="cuda")
    sA = torch.full((M, K // 32), 0x7F, dtype=torch.uint8, device="cuda")
    sB = torch.full((N, K // 32), 0x7F, dtype=torch.uint8, device="cuda")
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="static scratch"):
        ab.gemm_a8w8_mxfp8_noalloc(A, B, sA, sB, out, a_preshuffle=False, log2_k_split=4)
