"""The time-out path of the kernels, made to run without faulting or hanging anything: the wait limit is lowered to a
few milliseconds and one producer of a one-CTA problem is told to issue nothing (a flag nothing sets), so the waits
behind it run out.  The kernel must return by itself, leave a status record that names the wait, the next call must be
refused with that record's code until it has been fetched, and the launch after that must be healthy again."""
import pytest
import torch

from oracle import mx_oracle as ox
from tests.helpers import check, quant_fp8, randn_bf16, to_cuda_u8

pytestmark = pytest.mark.gpu

ST_TIMEOUT_CODES = {0x101, 0x102, 0x103, 0x104, 0x105, 0x106}


def _problem(ab, M, N, K, seed):
    x, w = randn_bf16(M, K, seed + 1), randn_bf16(N, K, seed + 2)
    xq, xs = quant_fp8(x)
    wq, ws = quant_fp8(w)
    ref = ox.gemm_a8w8_mxfp8_ref(xq, wq, xs, ws)
    args = (to_cuda_u8(xq, torch.float8_e4m3fn), ab.shuffle_mxfp8fp4_b(to_cuda_u8(wq, torch.float8_e4m3fn)),
            ab.shuffle_mxfp8fp4_scale(to_cuda_u8(xs)), ab.shuffle_mxfp8fp4_scale(to_cuda_u8(ws)))
    return ref, args


def test_a_wait_that_runs_out_is_reported_and_the_library_recovers():
    import aiter_b200 as ab

    M, N, K = 64, 128, 512  # one weight tile, no K split: a single CTA
    ref, args = _problem(ab, M, N, K, seed=70)
    out = ab.gemm_a8w8_mxfp8(*args, a_preshuffle=False, kernelName="tc5_128x64_t_s4_k0")
    check(ref, out, what="before the injected time-out")
    assert ab.device_status(0) == (0, 0, 0, 0)
    try:
        ab.debug_wait_control(0, limit_ns=3_000_000, withhold_scales=True)
        ab.gemm_a8w8_mxfp8(*args, a_preshuffle=False, kernelName="tc5_128x64_t_s4_k0")
        torch.cuda.synchronize()  # returns: the kernel gave up by itself after ~3 ms per wait
        # the failure surfaces at the caller's next call, before anything is launched
        launches = ab.launch_count()
        with pytest.raises(RuntimeError, match="gave up on a wait"):
            ab.gemm_a8w8_mxfp8(*args, a_preshuffle=False, kernelName="tc5_128x64_t_s4_k0")
        assert ab.launch_count() == launches
    finally:
        ab.debug_wait_control(0)  # defaults: 1 s, nothing withheld
    code, block, split, detail = ab.device_status(0)
    assert code in ST_TIMEOUT_CODES, hex(code)
    assert block == 0 and split == 0
    assert ab.device_status(0) == (0, 0, 0, 0)  # fetched and cleared
    # a split-K problem and the first problem again: tickets and barriers start clean
    ref2, args2 = _problem(ab, 16, 512, 4096, seed=71)
    out2 = ab.gemm_a8w8_mxfp8(*args2, a_preshuffle=False, kernelName="tc5_128x16_t_s4_k2")
    check(ref2, out2, what="split-K launch after the time-out")
    out = ab.gemm_a8w8_mxfp8(*args, a_preshuffle=False, kernelName="tc5_128x64_t_s4_k0")
    check(ref, out, what="after the injected time-out")
    assert ab.device_status(0) == (0, 0, 0, 0)
