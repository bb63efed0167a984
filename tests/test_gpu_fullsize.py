"""Parity at the benchmark's full sizes.  The oracle cannot finish a 4 TFLOP product in seconds, so each case checks
(a) 64 random rows of the output against the oracle run on exactly those activation rows (all N columns), and
(b) a size-independent property: adding 1 to every activation scale byte doubles every output element exactly
    (power-of-two scaling commutes with every rounding on the path), which exercises all tiles and all of K.
Inputs are seeded N(0,1) bf16 data, quantised on the GPU by the torch quantisers the CPU tests pin to the oracle."""
import numpy as np
import pytest
import torch

from helpers import check
from oracle import mx_oracle as ox

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def _rows(M, seed, n=64):
    g = np.random.default_rng(seed)
    return np.sort(g.choice(M, size=min(n, M), replace=False))


def _randn(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(rows, cols, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(16384, 7168, 16384), (16384, 24576, 1536), (16384, 7168, 7168)])
def test_mxfp4_full_size(ab, M, N, K):
    xq, xs = ab.per_1x32_f4_quant(_randn(M, K, 1))
    wq, ws = ab.per_1x32_f4_quant(_randn(N, K, 2))
    xs, ws = xs.view(torch.uint8), ws.view(torch.uint8)
    B = ab.shuffle_weight(wq.view(torch.uint8), layout=(16, 16))
    sB = ab.fp4_utils.e8m0_shuffle(ws)
    out = ab.gemm_a4w4(xq, B, ab.fp4_utils.e8m0_shuffle(xs), sB)
    assert out.shape == (M, N)
    rows = _rows(M, 3)
    ref = ox.gemm_a4w4_ref(xq.view(torch.uint8)[rows].cpu().numpy(), wq.view(torch.uint8).cpu().numpy(), xs[rows].cpu().numpy(), ws.cpu().numpy())
    check(ref, out[rows], what=f"gemm_a4w4 {M}x{N}x{K}, 64 rows")
    out2 = ab.gemm_a4w4(xq, B, ab.fp4_utils.e8m0_shuffle(xs + 1), sB)
    assert torch.equal(out2.float(), out.float() * 2.0)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_mxfp8_full_size(ab):
    M, N, K = 8192, 4096, 4096
    xq, xs = ab.per_1x32_f8_scale_f8_quant(_randn(M, K, 4), scale_type=ab.dtypes.fp8_e8m0)
    wq, ws = ab.per_1x32_f8_scale_f8_quant(_randn(N, K, 5), scale_type=ab.dtypes.fp8_e8m0)
    xs, ws = xs.view(torch.uint8), ws.view(torch.uint8)
    B, sB = ab.shuffle_mxfp8fp4_b(wq), ab.shuffle_mxfp8fp4_scale(ws)
    out = ab.gemm_a8w8_mxfp8(xq, B, ab.shuffle_mxfp8fp4_scale(xs), sB, a_preshuffle=False)
    rows = _rows(M, 6)
    ref = ox.gemm_a8w8_mxfp8_ref(xq.view(torch.uint8)[rows].cpu().numpy(), wq.view(torch.uint8).cpu().numpy(), xs[rows].cpu().numpy(), ws.cpu().numpy())
    check(ref, out[rows], what=f"gemm_a8w8_mxfp8 {M}x{N}x{K}, 64 rows")
    out2 = ab.gemm_a8w8_mxfp8(xq, B, ab.shuffle_mxfp8fp4_scale(xs + 1), sB, a_preshuffle=False)
    assert torch.equal(out2.float(), out.float() * 2.0)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_a8w4_full_size(ab):
    M, N, K = 16384, 8192, 8192
    xq, xs = ab.per_1x32_f8_scale_f8_quant(_randn(M, K, 7), scale_type=ab.dtypes.fp8_e8m0)
    wq, ws = ab.per_1x32_f4_quant(_randn(N, K, 8))
    xs, ws = xs.view(torch.uint8), ws.view(torch.uint8)
    B, sB = ab.shuffle_mxfp8fp4_b(wq.view(torch.uint8)), ab.shuffle_mxfp8fp4_scale(ws)
    out = ab.gemm_a8w4_mxfp8(xq, B, ab.shuffle_mxfp8fp4_scale(xs), sB, a_preshuffle=False)
    rows = _rows(M, 9)
    ref = ox.gemm_a8w4_mxfp8_ref(xq.view(torch.uint8)[rows].cpu().numpy(), wq.view(torch.uint8).cpu().numpy(), xs[rows].cpu().numpy(), ws.cpu().numpy())
    check(ref, out[rows], what=f"gemm_a8w4_mxfp8 {M}x{N}x{K}, 64 rows")
    out2 = ab.gemm_a8w4_mxfp8(xq, B, ab.shuffle_mxfp8fp4_scale(xs + 1), sB, a_preshuffle=False)
    assert torch.equal(out2.float(), out.float() * 2.0)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_nvfp4_full_size(ab):
    # the 8-GPU shard shape with NVFP4 inputs: random codes, e4m3 scales around 0.34, per-tensor factors; the
    # size-independent property here is linearity in a per-tensor factor (a power of two commutes with every rounding)
    M, N, K = 16384, 7168, 7168
    g = torch.Generator(device="cuda").manual_seed(10)
    xq = torch.randint(0, 256, (M, K // 2), generator=g, device="cuda", dtype=torch.uint8)
    wq = torch.randint(0, 256, (N, K // 2), generator=g, device="cuda", dtype=torch.uint8)
    xs = (torch.randn(M, K // 16, generator=g, device="cuda") * 0.08 + 0.34375).clamp(2.0 ** -6, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    ws = (torch.randn(N, K // 16, generator=g, device="cuda") * 0.08 + 0.34375).clamp(2.0 ** -6, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    A, B = ab.shuffle_weight_f4(xq), ab.shuffle_weight_f4(wq)
    sA, sB = ab.shuffle_scale_f4(xs, 8), ab.shuffle_scale_f4(ws, 8)
    out = ab.gemm_nvfp4_asm(A, B, sA, sB, 0.75, 1.25, a_preshuffle=True)
    assert out.shape == (M, N)
    rows = _rows(M, 11)
    ref = ox.gemm_nvfp4_ref(xq[rows].cpu().numpy(), wq.cpu().numpy(), xs[rows].cpu().numpy(), ws.cpu().numpy(), 0.75, 1.25)
    check(ref, out[rows], what=f"gemm_nvfp4_asm {M}x{N}x{K}, 64 rows")
    out2 = ab.gemm_nvfp4_asm(A, B, sA, sB, 1.5, 1.25, a_preshuffle=True)
    assert torch.equal(out2.float(), out.float() * 2.0)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_bf16_full_size(ab):
    # 8192^3: 64 rows against the oracle; property: doubling the activations doubles the output exactly
    M = N = K = 8192
    a, b = _randn(M, K, 10) * 0.1, _randn(N, K, 11) * 0.1
    a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
    out = ab.tgemm.mm(a, b)
    rows = _rows(M, 12)
    ref = ox.gemm_a16w16_ref(a[rows].cpu().view(torch.int16).numpy().view(np.uint16), b.cpu().view(torch.int16).numpy().view(np.uint16))
    check(ref, out[rows], what="bf16 8192^3, 64 rows")
    assert torch.equal(ab.tgemm.mm(a * 2, b).float(), out.float() * 2.0)
    assert ab.device_status(0) == (0, 0, 0, 0)
