"""NVFP4 inputs of the F4GEMM entry point (packed e2m1 data, one e4m3 scale per 16 elements, two per-tensor factors)
against the numpy oracle: bf16, packed-fp4 and mxfp8 outputs, every tile family, the K splits, and the reference's
constant known-answer case."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as ox
from tests.helpers import check, to_cuda_u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def _pad_rows(s: np.ndarray, fill: int) -> np.ndarray:
    rows = (s.shape[0] + 31) // 32 * 32
    out = np.full((rows, s.shape[1]), fill, dtype=np.uint8)
    out[: s.shape[0]] = s
    return out


def _problem(M, N, K, seed, scales="gauss"):
    """Random e2m1 codes; e4m3 scales drawn as the reference's bench initialiser does (normal(0.34375, 0.08), positive),
    or powers of two (exact fp32 sums), or all 1.0."""
    g = np.random.default_rng(seed)
    xq = g.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    wq = g.integers(0, 256, size=(N, K // 2), dtype=np.uint8)

    def sc(rows):
        if scales == "gauss":
            return ox.f32_to_e4m3fn(np.clip(g.normal(0.34375, 0.08, size=(rows, K // 16)), 2.0 ** -6, 448.0).astype(np.float32))
        if scales == "pow2":
            return g.choice(np.array([0x30, 0x38, 0x40], dtype=np.uint8), size=(rows, K // 16))  # 0.5, 1, 2
        return np.full((rows, K // 16), 0x38, dtype=np.uint8)

    return xq, wq, sc(M), sc(N)


def _operands(ab, xq, wq, xs, ws, apre):
    A = to_cuda_u8(xq)
    return (ab.shuffle_weight_f4(A) if apre else A, ab.shuffle_weight_f4(to_cuda_u8(wq)),
            ab.shuffle_scale_f4(to_cuda_u8(_pad_rows(xs, 0x38)), 8), ab.shuffle_scale_f4(to_cuda_u8(_pad_rows(ws, 0x38)), 8))


@pytest.mark.parametrize("M,N,K,apre,name", [
    (32, 128, 256, 0, ""), (1, 256, 512, 0, ""), (20, 384, 768, 0, ""), (192, 384, 512, 1, ""), (512, 1024, 1024, 1, ""),
    (64, 512, 2048, 0, "tc5_128x64_t_s4_k2"),   # weights on the 128-row slot, K split over a cluster
    (16, 256, 4096, 0, "tc5_128x16_t_s0_k3"),   # (eight slices: the persistent kernel)
    (8, 640, 2048, 0, "tc5_128x16_t_s3_k2"),    # decode kernel
    (200, 384, 512, 0, "tc5_128x64_t_s0_k1"),   # decode kernel, four tiles of 64 rows, ragged
    (256, 256, 1024, 1, "tc5_128x128_t_s0_k0"), # decode kernel, two tiles of 128 rows
    (300, 640, 512, 0, "tc5_128x128_n_s0"),     # ragged rows and a ragged last tile
    (300, 640, 1024, 0, "tc5_128x64_n_s3_k1"),  # workspace K split
    (1024, 768, 512, 1, "tc5_256x256_n_s0"),    # CTA pair
    (1024, 1024, 768, 0, "tc5_256x192_n_s0"),
    (640, 512, 256, 0, "tc5_128x256_n_s2"),
])
def test_nvfp4_bf16_output(ab, M, N, K, apre, name):
    xq, wq, xs, ws = _problem(M, N, K, seed=M + N + K)
    ga, gb = 0.75, 1.3
    ref = ox.gemm_nvfp4_ref(xq, wq, xs, ws, ga, gb)
    before = ab.launch_count()
    out = ab.gemm_nvfp4_asm(*_operands(ab, xq, wq, xs, ws, apre), ga, gb, a_preshuffle=bool(apre), kernelName=name)
    assert ab.launch_count() > before
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    check(ref, out, what=f"nvfp4 {M}x{N}x{K} apre={apre} {name or 'heuristic'}")
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_nvfp4_constant_known_answer(ab):
    # op_tests/test_f4gemm.py:169-178: A = 0x22 (1.0), B = 0x33 (1.5), scales 0x38 (1.0) -> every output 1.5 * K
    M, N, K = 64, 256, 512
    xq = np.full((M, K // 2), 0x22, dtype=np.uint8)
    wq = np.full((N, K // 2), 0x33, dtype=np.uint8)
    one = lambda rows: np.full((rows, K // 16), 0x38, dtype=np.uint8)  # noqa: E731
    out = ab.gemm_nvfp4_asm(*_operands(ab, xq, wq, one(M), one(N), 0), 1.0, 1.0, a_preshuffle=False)
    assert (out.float().cpu().numpy() == 1.5 * K).all()
    out = ab.gemm_nvfp4_asm(*_operands(ab, xq, wq, one(M), one(N), 1), 0.5, 0.25, a_preshuffle=True)
    assert (out.float().cpu().numpy() == 1.5 * K / 8).all()
    # every scale byte matters: one block of one weight row at 2.0 adds 16 products of 1.5 to that column
    ws = one(N)
    ws[5, 3] = 0x40
    out = ab.gemm_nvfp4_asm(*_operands(ab, xq, wq, one(M), ws, 0), 1.0, 1.0, a_preshuffle=False).float().cpu().numpy()
    want = np.full((M, N), 1.5 * K, dtype=np.float32)
    want[:, 5] += 16 * 1.5
    assert (out == want).all()
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_gemm_a4w4_with_global_scales_is_nvfp4(ab):
    M, N, K = 96, 256, 512
    xq, wq, xs, ws = _problem(M, N, K, seed=11)
    A, B, sA, sB = _operands(ab, xq, wq, xs, ws, 0)
    ga, gb = torch.tensor([0.5]), torch.tensor(1.25, device="cuda")
    out = ab.gemm_a4w4(A.view(2, M // 2, K // 2), B, sA, sB, global_A_scale=ga, global_B_scale=gb)
    assert out.shape == (2, M // 2, N)
    check(ox.gemm_nvfp4_ref(xq, wq, xs, ws, 0.5, 1.25), out.view(M, N), what="gemm_a4w4 with global scales")
    # one global scale alone selects NVFP4 too; the other is 1
    out = ab.gemm_a4w4(A, B, sA, sB, global_B_scale=2.0)
    check(ox.gemm_nvfp4_ref(xq, wq, xs, ws, 1.0, 2.0), out, what="gemm_a4w4 with one global scale")
    assert ab.device_status(0) == (0, 0, 0, 0)


@pytest.mark.parametrize("M,N,K,apre", [(64, 128, 256, 0), (192, 384, 512, 1), (512, 1024, 256, 0)])
def test_nvfp4_low_precision_outputs_bit_exact_on_exact_sums(ab, M, N, K, apre):
    # power-of-two scales and factors: every partial sum is exact in fp32, so the re-quantised bytes must be identical
    xq, wq, xs, ws = _problem(M, N, K, seed=M + 1, scales="pow2")
    ga, gb = 0.5, 4.0
    ops = _operands(ab, xq, wq, xs, ws, apre)
    ref_q, ref_s = ox.requant_mxfp8_blockN(ox.gemm_nvfp4_f32(xq, wq, xs, ws, ga, gb))
    out, scale = ab.gemm_a4w4o8(*ops, apreshuffle=bool(apre), global_A_scale=ga, global_B_scale=gb)
    assert np.array_equal(ab.unpack_mxfp8_out_scale(scale, M, N).view(torch.uint8).cpu().numpy(), ref_s), "scale bytes differ"
    assert np.array_equal(out.view(torch.uint8).cpu().numpy(), ref_q), "e4m3 codes differ"
    # packed fp4: the block scales are dropped, the per-tensor factors stay (op_tests/test_f4gemm.py:125-129)
    xq3 = xq & 0x33
    ops = _operands(ab, xq3, wq, xs, ws, apre)
    ref4 = ox.requant_fp4(ox.gemm_nvfp4_f32(xq3, wq, xs, ws, 0.25, 0.5, noscale=True))
    out4 = ab.gemm_a4w4o4(*ops, apreshuffle=bool(apre), global_A_scale=0.25, global_B_scale=0.5)
    assert out4.shape == (M, N // 2)
    assert np.array_equal(out4.view(torch.uint8).cpu().numpy(), ref4)
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_nvfp4_refuses_what_it_cannot_serve(ab):
    xq, wq, xs, ws = _problem(32, 128, 256, seed=3)
    A, B, sA, sB = _operands(ab, xq, wq, xs, ws, 0)
    with pytest.raises(RuntimeError, match="256"):
        ab.gemm_nvfp4_asm(A[:, :64].contiguous(), B[:, :64].contiguous(), sA, sB, 1.0, 1.0, a_preshuffle=False)  # K = 128
    with pytest.raises(RuntimeError, match="columns"):
        ab.gemm_nvfp4_asm(A, B, sA[:, :8].contiguous(), sB, 1.0, 1.0, a_preshuffle=False)  # K/32 scales: the MXFP4 count
    with pytest.raises(RuntimeError, match="not find kernel"):
        ab.gemm_nvfp4_asm(A, B, sA, sB, 1.0, 1.0, a_preshuffle=False, kernelName="no_such_kernel")
    assert ab.device_status(0) == (0, 0, 0, 0)
