"""Output forms beside bf16: fp32 straight from the accumulator, fp16, a batch as one launch, and the re-quantising
epilogues of the MXFP4 GEMM (packed e2m1; e4m3 + one UE8M0 scale per 128 columns), against the numpy oracle."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as ox
from tests.helpers import bf16_bits, check, quant_fp4, randn_bf16, to_cuda_u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def _f4_operands(ab, xq, wq, xs, ws, apre):
    A = to_cuda_u8(xq)
    return (ab.shuffle_weight_f4(A) if apre else A, ab.shuffle_weight_f4(to_cuda_u8(wq)),
            ab.shuffle_scale_f4(to_cuda_u8(xs)), ab.shuffle_scale_f4(to_cuda_u8(ws)))


def _exact_problem(M, N, K, seed):
    """Packed e2m1 codes and power-of-two scales for which every partial sum is exact in fp32 whatever the order of
    accumulation: the tensor core's and numpy's fp32 products are then the same numbers, and the re-quantised outputs
    can be compared bit for bit."""
    g = np.random.default_rng(seed)
    xq = g.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    wq = g.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    xs = g.integers(126, 129, size=(M, K // 32), dtype=np.uint8)
    ws = g.integers(126, 129, size=(N, K // 32), dtype=np.uint8)
    return xq, wq, xs, ws


@pytest.mark.parametrize("M,N,K,apre", [(64, 128, 256, 0), (192, 384, 512, 1), (512, 1024, 256, 0), (640, 768, 1024, 1)])
def test_gemm_a4w4o8_bit_exact_on_exact_sums(ab, M, N, K, apre):
    xq, wq, xs, ws = _exact_problem(M, N, K, seed=M + N)
    ref_q, ref_s = ox.gemm_a4w4o8_ref(xq, wq, xs, ws)
    out, scale = ab.gemm_a4w4o8(*_f4_operands(ab, xq, wq, xs, ws, apre), apreshuffle=bool(apre))
    assert out.shape == (M, N) and out.dtype == ab.dtypes.fp8 and scale.shape == (M, N // 128)
    got_s = ab.unpack_mxfp8_out_scale(scale, M, N).view(torch.uint8).cpu().numpy()
    assert np.array_equal(got_s, ref_s), "scale bytes differ"
    assert np.array_equal(scale.view(torch.uint8).cpu().numpy().reshape(-1), ox.pack_mxfp8_out_scale(ref_s).reshape(-1)), "packed scale order"
    assert np.array_equal(out.view(torch.uint8).cpu().numpy(), ref_q), "e4m3 codes differ"
    assert ab.device_status(0) == (0, 0, 0, 0)


@pytest.mark.parametrize("M,N,K,apre", [(64, 128, 256, 0), (192, 384, 512, 1), (512, 1024, 256, 0)])
def test_gemm_a4w4o4_bit_exact_on_exact_sums(ab, M, N, K, apre):
    xq, wq, xs, ws = _exact_problem(M, N, K, seed=M + N + 1)
    xq &= 0x33  # codes 0..3 and no sign: |values| <= 1.5, so the sums spread over the e2m1 range instead of saturating
    ref = ox.gemm_a4w4o4_ref(xq, wq)  # the block scales are not applied, as in the reference's fp4-output kernel
    out = ab.gemm_a4w4o4(*_f4_operands(ab, xq, wq, xs, ws, apre), apreshuffle=bool(apre))
    assert out.shape == (M, N // 2)
    assert np.array_equal(out.view(torch.uint8).cpu().numpy(), ref)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_gemm_a4w4o8_random_data_within_the_references_tolerance(ab):
    # seeded N(0,1) data: fp32 sums differ in the last bit between accumulation orders, so the comparison is the
    # reference test's own (op_tests/test_f4gemm.py:385-404): scale bytes within 1, dequantised data rtol 0.1 / atol 1
    M, N, K = 256, 512, 1024
    xq, xs = quant_fp4(randn_bf16(M, K, 21))
    wq, ws = quant_fp4(randn_bf16(N, K, 22))
    ref_q, ref_s = ox.gemm_a4w4o8_ref(xq, wq, xs, ws)
    out, scale = ab.gemm_a4w4o8(*_f4_operands(ab, xq, wq, xs, ws, 0))
    got_s = ab.unpack_mxfp8_out_scale(scale, M, N).view(torch.uint8).cpu().numpy()
    assert np.abs(got_s.astype(np.int32) - ref_s.astype(np.int32)).max() <= 1
    deq = lambda q, s: ox.e4m3fn_to_f32(q).reshape(M, N // 128, 128) * ox.e8m0_to_f32(s)[:, :, None]  # noqa: E731
    a, b = deq(ref_q, ref_s), deq(out.view(torch.uint8).cpu().numpy(), got_s)
    assert np.all(np.abs(a - b) <= 1.0 + 0.1 * np.abs(a))
    assert (got_s == ref_s).mean() > 0.99 and (out.view(torch.uint8).cpu().numpy() == ref_q).mean() > 0.98


def test_low_precision_outputs_refuse_what_they_cannot_serve(ab):
    xq, wq, xs, ws = _exact_problem(64, 192, 256, seed=5)  # N % 128 != 0
    with pytest.raises((RuntimeError, AssertionError)):
        ab.gemm_a4w4o8(*_f4_operands(ab, xq, wq, xs, ws, 0))
    with pytest.raises(NotImplementedError, match="gemm_a4w4o4"):
        A, B, sA, sB = _f4_operands(ab, *_exact_problem(64, 128, 256, 6), 0)
        ab.gemm_a4w4(A, B, sA, sB, dtype=ab.dtypes.fp4x2)  # one plain tensor only: the low-precision forms have their own entry points


# ------------------------------------------------------------------------------------------- bf16: fp32 output, batch
@pytest.mark.parametrize("M,N,K", [(64, 1024, 1024), (3, 512, 1024), (300, 1000, 264), (8, 256, 8192), (700, 768, 2048)])
def test_bf16_fp32_output(ab, M, N, K):
    a, b = randn_bf16(M, K, 31, 0.1), randn_bf16(N, K, 32, 0.1)
    ref = ox.gemm_f32(ox.bf16_bits_to_f32(bf16_bits(a)), ox.bf16_bits_to_f32(bf16_bits(b)))
    for out in (ab.gemm_a16w16_opus(a.cuda(), b.cuda(), dtype=torch.float32), ab.tgemm.mm(a.cuda(), b.cuda(), otype=torch.float32)):
        assert out.dtype == torch.float32 and out.shape == (M, N)
        got = out.cpu().numpy()
        # no bf16 rounding on the way out: two fp32 accumulations of K products agree far inside the bf16 grid
        assert np.all(np.abs(got - ref) <= 1e-4 + 1e-4 * np.abs(ref)), np.abs(got - ref).max()
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_bf16_batch_is_one_launch(ab):
    batch, M, N, K = 4, 40, 320, 512
    a = randn_bf16(batch * M, K, 33, 0.1).view(batch, M, K)
    b = randn_bf16(batch * N, K, 34, 0.1).view(batch, N, K)
    bias = randn_bf16(batch, N, 35).float()
    for dtype in (torch.bfloat16, torch.float32):
        before = ab.launch_count()
        out = ab.gemm_a16w16_opus(a.cuda(), b.cuda(), bias=bias.cuda(), dtype=dtype)
        assert ab.launch_count() == before + 1, "the batch must be one launch"
        assert out.shape == (batch, M, N) and out.dtype == dtype
        for i in range(batch):
            ref = ox.gemm_f32(ox.bf16_bits_to_f32(bf16_bits(a[i])), ox.bf16_bits_to_f32(bf16_bits(b[i]))) + bias[i].numpy()[None, :]
            if dtype == torch.float32:
                assert np.all(np.abs(out[i].cpu().numpy() - ref) <= 1e-4 + 1e-4 * np.abs(ref))
            else:
                check(ox.f32_to_bf16_bits(ref.astype(np.float32)), out[i], what=f"batch entry {i}")
    # a split-K kernel id on a batch: tickets and partial tiles are per (entry, tile)
    y = torch.full((batch, M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    before = ab.launch_count()
    ab.opus_gemm_a16w16_tune(a.cuda(), b.cuda(), y, None, 20, 2)
    assert ab.launch_count() == before + 1
    for i in range(batch):
        check(ox.gemm_a16w16_ref(bf16_bits(a[i]), bf16_bits(b[i])), y[i], what=f"split-K batch entry {i}")
    assert ab.device_status(0) == (0, 0, 0, 0)


# ------------------------------------------------------------------------------------------- fp8 blockscale: fp16 / fp32 output
def _blockscale_problem(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * 2).to(torch.float8_e4m3fn)
    w = (torch.randn(N, K, generator=g) * 2).to(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, generator=g) + 0.25
    ws = torch.rand((N + 127) // 128, K // 128, generator=g) + 0.25
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), xs.numpy(), ws.numpy())
    return x, w, xs, ws, ox.bf16_bits_to_f32(ref)


@pytest.mark.parametrize("M", [16, 100, 700])
def test_blockscale_fp16_output_and_opus_scaled_fp32(ab, M):
    N, K = 512, 1024
    x, w, xs, ws, ref = _blockscale_problem(M, N, K, seed=40 + M)
    out = ab.gemm_a8w8_blockscale(x.cuda(), w.cuda(), xs.cuda(), ws.cuda(), dtype=torch.float16)
    assert out.dtype == torch.float16
    got = out.float().cpu().numpy()
    assert np.all(np.abs(got - ref) <= 1e-2 + 1e-2 * np.abs(ref))
    # the same product through opus_gemm's scaled form: fp8 operands, fp32 scales, fp32 output
    y = torch.empty((1, M, N), dtype=torch.float32, device="cuda")
    ab.opus_gemm(x.cuda()[None], w.cuda()[None], y, None, xs.cuda()[None], ws.cuda()[None], None)
    assert np.all(np.abs(y[0].cpu().numpy() - ref) <= 1e-2 + 1e-2 * np.abs(ref))
    assert ab.device_status(0) == (0, 0, 0, 0)
