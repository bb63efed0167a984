"""CUDA path vs the numpy oracle, through the operator surface and the C ABI (needs a B200)."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as ox
from tests.helpers import bf16_bits, check, quant_fp4, quant_fp8, randn_bf16, to_cuda_u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def assert_healthy(ab):
    st = ab.device_status(0)
    assert st == (0, 0, 0, 0), f"kernel recorded an expired wait: {[hex(w) for w in st]}"


# ------------------------------------------------------------------------------------------- bf16
BF16_SHAPES = [
    (64, 1024, 1024),  # the reference's own CPU-runnable case
    (1, 256, 512), (3, 512, 1024), (16, 1024, 4096), (33, 384, 520), (127, 272, 1032), (129, 512, 512),
    (300, 1000, 264), (512, 2048, 2048),
]


@pytest.mark.parametrize("M,N,K", BF16_SHAPES)
def test_bf16_tgemm(ab, M, N, K):
    a = randn_bf16(M, K, 1, 0.1)
    b = randn_bf16(N, K, 2, 0.1)
    ref = ox.gemm_a16w16_ref(bf16_bits(a), bf16_bits(b))
    out = ab.tgemm.mm(a.cuda(), b.cuda())
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    check(ref, out, what=f"tgemm.mm {M}x{N}x{K}")
    assert_healthy(ab)


@pytest.mark.parametrize("kernel_id,log2_split", [(100, 0), (100, 2), (113, 1), (120, 3), (20, 0), (32, 1), (30, 2), (40, 0), (44, 1), (140, 0),
                                                  (50, 0), (60, 1), (70, 0), (80, 0), (1040, 0), (1030, 1), (1053, 0), (1060, 0), (1130, 0)])
def test_bf16_every_tile_shape(ab, kernel_id, log2_split):
    M = 16 if kernel_id == 100 else (600 if kernel_id >= 1000 else 200)
    N, K = 768, 2048
    a = randn_bf16(M, K, 3, 0.1)
    b = randn_bf16(N, K, 4, 0.1)
    bias = randn_bf16(1, N, 5).view(-1)
    ref = ox.gemm_a16w16_ref(bf16_bits(a), bf16_bits(b), bias.float().numpy())
    y = torch.full((1, M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ab.opus_gemm_a16w16_tune(a.cuda()[None], b.cuda()[None], y, bias.cuda(), kernel_id, log2_split)
    check(ref, y[0], what=f"kernelId {kernel_id} splitK 2^{log2_split}")
    assert_healthy(ab)


def test_bf16_split_k_twice_in_a_row(ab):
    # the ticket counters must be back at zero after a launch
    a = randn_bf16(8, 8192, 6, 0.1)
    b = randn_bf16(256, 8192, 7, 0.1)
    ref = ox.gemm_a16w16_ref(bf16_bits(a), bf16_bits(b))
    for _ in range(3):
        y = torch.zeros((1, 8, 256), dtype=torch.bfloat16, device="cuda")
        ab.opus_gemm_a16w16_tune(a.cuda()[None], b.cuda()[None], y, None, 100, 4)
        check(ref, y[0], what="split-K x16 repeat")
    assert_healthy(ab)


def test_bf16_shuffled_weight_and_batch(ab):
    a = randn_bf16(2 * 40, 512, 8, 0.1).view(2, 40, 512)
    b = randn_bf16(320, 512, 9, 0.1)
    ref = ox.gemm_a16w16_ref(bf16_bits(a.view(80, 512)), bf16_bits(b)).reshape(2, 40, 320)
    bs = ab.shuffle_weight(b.cuda(), layout=(16, 16))
    assert bs.is_shuffled
    out = ab.gemm_a16w16(a.cuda(), bs)
    check(ref.reshape(80, 320), out.view(80, 320), what="shuffled weight, 3-D activations")
    out2 = ab.gemm_a16w16_opus(a.cuda(), b.cuda()[None].expand(2, -1, -1).contiguous())
    check(ref.reshape(80, 320), out2.reshape(80, 320), what="opus batched")
    assert_healthy(ab)


def test_bf16_padded_row_pitch(ab):
    big = randn_bf16(70, 1024 + 64, 10, 0.1).cuda()
    a = big[:, :1024]  # row pitch 1088 elements
    b = randn_bf16(128, 1024, 11, 0.1)
    ref = ox.gemm_a16w16_ref(bf16_bits(a), bf16_bits(b))
    y = torch.empty((1, 70, 128), dtype=torch.bfloat16, device="cuda")
    ab.opus_gemm(a[None], b.cuda()[None], y)
    check(ref, y[0], what="padded lda")
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- MXFP8
def mxfp8_case(ab, M, N, K, apre, seed=0):
    x, w = randn_bf16(M, K, seed + 1), randn_bf16(N, K, seed + 2)
    xq, xs = quant_fp8(x)
    wq, ws = quant_fp8(w)
    ref = ox.gemm_a8w8_mxfp8_ref(xq, wq, xs, ws)
    A = to_cuda_u8(xq, torch.float8_e4m3fn)
    if apre:
        A = ab.shuffle_mxfp8fp4_a(A)
    B = ab.shuffle_mxfp8fp4_b(to_cuda_u8(wq, torch.float8_e4m3fn))
    sA = ab.shuffle_mxfp8fp4_scale(to_cuda_u8(xs))
    sB = ab.shuffle_mxfp8fp4_scale(to_cuda_u8(ws))
    return ref, (A, B, sA, sB)


@pytest.mark.parametrize("M,N,K,apre", [
    (1, 256, 128, 0), (16, 512, 1024, 0), (16, 512, 1024, 1), (128, 4096, 4096, 1), (130, 304, 640, 1),
    (300, 1024, 2048, 0), (1024, 512, 512, 1), (33, 4096, 4096, 0),
])
def test_mxfp8(ab, M, N, K, apre):
    ref, args = mxfp8_case(ab, M, N, K, apre)
    out = ab.gemm_a8w8_mxfp8(*args, a_preshuffle=bool(apre))
    check(ref, out, what=f"gemm_a8w8_mxfp8 {M}x{N}x{K} apre={apre}")
    assert_healthy(ab)


@pytest.mark.parametrize("name", ["tc5_128x16_t_s4", "tc5_128x32_t_s3", "tc5_128x64_t_s2", "tc5_128x128_t_s4",
                                  "tc5_128x32_n_s4", "tc5_128x64_n_s4", "tc5_128x128_n_s4", "tc5_128x256_n_s4",
                                  "tc5_128x192_n_s4", "tc5_128x224_n_s3", "tc5_128x96_n_s4", "tc5_128x160_n_s4",
                                  "tc5_256x256_n_s4", "tc5_256x128_n_s6", "tc5_256x192_n_s5", "tc5_256x224_n_s4", "tc5_256x64_n_s4"])
def test_mxfp8_every_tile_shape(ab, name):
    M = 16 if "x16_" in name else (700 if name.startswith("tc5_256") else 160)
    ref, args = mxfp8_case(ab, M, 768, 1536, 0, seed=5)
    out = ab.gemm_a8w8_mxfp8(*args, a_preshuffle=False, kernelName=name)
    check(ref, out, what=name)
    assert_healthy(ab)


def test_mxfp8_constant_known_answer(ab):
    # A = B = 0.5, unit scales: every output is 0.25 * K
    M, N, K = 64, 256, 512
    A = torch.full((M, K), 0.5).to(torch.float8_e4m3fn).cuda()
    B = ab.shuffle_mxfp8fp4_b(torch.full((N, K), 0.5).to(torch.float8_e4m3fn).cuda())
    s = torch.full((M, K // 32), 0x7F, dtype=torch.uint8).cuda()
    sb = torch.full((N, K // 32), 0x7F, dtype=torch.uint8).cuda()
    out = ab.gemm_a8w8_mxfp8(A, B, ab.shuffle_mxfp8fp4_scale(s), ab.shuffle_mxfp8fp4_scale(sb), a_preshuffle=False)
    assert (out.float() == 0.25 * K).all()
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- MXFP4
def mxfp4_case(ab, M, N, K, seed=0):
    x, w = randn_bf16(M, K, seed + 1), randn_bf16(N, K, seed + 2)
    xq, xs = quant_fp4(x)
    wq, ws = quant_fp4(w)
    ref = ox.gemm_a4w4_ref(xq, wq, xs, ws)
    return ref, xq, wq, xs, ws


@pytest.mark.parametrize("M,N,K,bpre", [
    (1, 256, 256, True), (32, 512, 1024, True), (32, 512, 1024, False), (256, 7168, 2048, True), (100, 304, 320, True),
    (129, 1024, 1536, True), (17, 2048, 4096, True), (512, 512, 768, False),
])
def test_mxfp4_gemm_a4w4(ab, M, N, K, bpre):
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K)
    A = to_cuda_u8(xq, ab.dtypes.fp4x2)
    B = to_cuda_u8(wq)
    if bpre:
        B = ab.shuffle_weight(B, layout=(16, 16))
    sA = ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs))
    sB = ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws))
    out = ab.gemm_a4w4(A, B, sA, sB, bpreshuffle=bpre)
    assert out.shape == (M, N)
    check(ref, out, what=f"gemm_a4w4 {M}x{N}x{K} bpre={bpre}")
    assert_healthy(ab)


@pytest.mark.parametrize("kernel_id,log2_split", [(100, 0), (110, 2), (123, 1), (132, 0), (14, 1), (24, 0), (34, 2), (42, 0),
                                                  (52, 0), (62, 0), (1040, 0), (1044, 1), (1030, 0), (1050, 0), (1060, 0)])
def test_mxfp4_every_tile_shape(ab, kernel_id, log2_split):
    M = 16 if kernel_id == 100 else (520 if kernel_id >= 1000 else 192)
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, 512, 2048, seed=7)
    out = torch.full((M, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    ab.gemm_a4w4_blockscale_tune(
        to_cuda_u8(xq), ab.shuffle_weight(to_cuda_u8(wq)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs)),
        ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws)), out, kernel_id, log2_split)
    check(ref, out, what=f"a4w4 kernelId {kernel_id} splitK 2^{log2_split}")
    assert_healthy(ab)


def test_mxfp4_alpha_bias(ab):
    M, N, K = 48, 256, 512
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K, seed=9)
    bias = torch.randn(1, N, generator=torch.Generator().manual_seed(3))
    want = ox.f32_to_bf16_bits((0.5 * ox.bf16_bits_to_f32(ox.gemm_a4w4_ref(xq, wq, xs, ws)) + 2.0 * bias.numpy()).astype(np.float32))
    out = torch.empty((64, N), dtype=torch.bfloat16, device="cuda")
    ab.gemm_a4w4_asm(to_cuda_u8(xq), ab.shuffle_weight(to_cuda_u8(wq)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs)),
                     ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws)), out, "", bias.cuda(), 0.5, 2.0, True)
    check(want, out[:M], rtol=2e-2, atol=2e-2, what="alpha/beta/bias")  # the oracle rounds to bf16 before scaling
    assert_healthy(ab)


@pytest.mark.parametrize("M,name", [(300, "tc5_128x128_n_s0"), (1024, "tc5_256x256_n_s0"), (700, "tc5_128x64_n_s3"), (200, "tc5_128x32_n_s3")])
def test_mxfp4_alpha_bias_on_row_major_tiles(ab, M, name):
    # the wide (64 columns per step) and narrow epilogues of tiles that keep the activations on the 128-row slot: alpha
    # alone, and alpha with a bias per output column
    N, K = 512, 512
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K, seed=M)
    args = (to_cuda_u8(xq), ab.shuffle_weight(to_cuda_u8(wq)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws)))
    bias = torch.randn(1, N, generator=torch.Generator().manual_seed(4))
    base = ox.bf16_bits_to_f32(ref)
    out = torch.full(((M + 31) // 32 * 32, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ab.gemm_a4w4_asm(*args, out, name, None, 0.25, 0.0, True)
    check(ox.f32_to_bf16_bits((0.25 * base).astype(np.float32)), out[:M], rtol=2e-2, atol=2e-2, what=f"alpha only, {name}")
    ab.gemm_a4w4_asm(*args, out, name, bias.cuda(), 0.5, 2.0, True)
    check(ox.f32_to_bf16_bits((0.5 * base + 2.0 * bias.numpy()).astype(np.float32)), out[:M], rtol=2e-2, atol=2e-2, what=f"alpha, beta, bias, {name}")
    assert_healthy(ab)


def test_mxfp4_g1250_scale_layout(ab):
    M, N, K = 64, 512, 1024
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K, seed=11)
    # the F4GEMM entry point takes both operands as 16x16-byte tiles (op_tests/test_f4gemm.py:155-158)
    for apre in (True, False):
        A = to_cuda_u8(xq)
        out = ab.gemm_mxfp4_asm(
            ab.shuffle_weight_f4(A) if apre else A, ab.shuffle_weight_f4(to_cuda_u8(wq)),
            ab.shuffle_scale_f4(to_cuda_u8(xs)), ab.shuffle_scale_f4(to_cuda_u8(ws)), a_preshuffle=apre)
        check(ref, out, what=f"mxfp4_gemm_asm a_preshuffle={apre}")
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- mixed MXFP8 x MXFP4
def a8w4_case(ab, M, N, K, apre, seed=0):
    x, w = randn_bf16(M, K, seed + 1), randn_bf16(N, K, seed + 2)
    xq, xs = quant_fp8(x)
    wq, ws = quant_fp4(w)
    ref = ox.gemm_a8w4_mxfp8_ref(xq, wq, xs, ws)
    A = to_cuda_u8(xq, torch.float8_e4m3fn)
    if apre:
        A = ab.shuffle_mxfp8fp4_a(A)
    B = ab.shuffle_mxfp8fp4_b(to_cuda_u8(wq))
    return ref, (A, B, ab.shuffle_mxfp8fp4_scale(to_cuda_u8(xs)), ab.shuffle_mxfp8fp4_scale(to_cuda_u8(ws)))


@pytest.mark.parametrize("M,N,K,apre", [
    (1, 256, 128, 0), (2, 512, 1024, 1), (16, 512, 1024, 0), (64, 1024, 2048, 1), (128, 8192, 8192, 1), (300, 1024, 2048, 0),
    (1024, 2048, 1024, 1), (130, 304, 640, 1),
])
def test_a8w4_mxfp8(ab, M, N, K, apre):
    ref, args = a8w4_case(ab, M, N, K, apre, seed=13)
    out = ab.gemm_a8w4_mxfp8(*args, a_preshuffle=bool(apre))
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    check(ref, out, what=f"gemm_a8w4_mxfp8 {M}x{N}x{K} apre={apre}")
    assert_healthy(ab)


@pytest.mark.parametrize("name", ["tc5_128x16_t_s4", "tc5_128x64_t_s3", "tc5_128x128_n_s4", "tc5_128x256_n_s3", "tc5_256x256_n_s4",
                                  "tc5_256x128_n_s5", "tc5_256x192_n_s4"])
def test_a8w4_every_tile_shape(ab, name):
    M = 16 if "x16_" in name else (600 if name.startswith("tc5_256") else 64 if "_t_" in name else 200)
    ref, args = a8w4_case(ab, M, 768, 1536, 0, seed=15)
    out = ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False, kernelName=name)
    check(ref, out, what=name)
    assert_healthy(ab)


def test_a8w4_tall_problem_takes_the_widening_prepass(ab):
    # M >= 1024: the packed e2m1 weight is widened to e4m3 once (one extra launch) and the GEMM runs as MXFP8;
    # the result must match the in-kernel path's oracle all the same, twice in a row (buffer re-use)
    M, N, K = 1024, 512, 1024
    ref, args = a8w4_case(ab, M, N, K, 0, seed=21)
    before = ab.launch_count()
    out = ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False)
    assert ab.launch_count() == before + 2
    check(ref, out, what="a8w4 with widening pre-pass")
    check(ref, ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False), what="a8w4 with widening pre-pass, second call")
    assert_healthy(ab)


def test_a8w4_constant_known_answer(ab):
    # A = 0.5 (e4m3), B nibbles 0x1 = 0.5 (e2m1), unit scales: every output is 0.25 * K
    M, N, K = 32, 256, 512
    A = torch.full((M, K), 0.5).to(torch.float8_e4m3fn).cuda()
    B = ab.shuffle_mxfp8fp4_b(torch.full((N, K // 2), 0x11, dtype=torch.uint8).cuda())
    sa = ab.shuffle_mxfp8fp4_scale(torch.full((M, K // 32), 0x7F, dtype=torch.uint8).cuda())
    sb = ab.shuffle_mxfp8fp4_scale(torch.full((N, K // 32), 0x7F, dtype=torch.uint8).cuda())
    out = ab.gemm_a8w4_mxfp8(A, B, sa, sb, a_preshuffle=False)
    assert (out.float() == 0.25 * K).all()
    assert_healthy(ab)


def test_a8w4_table_dispatch(ab, tmp_path, monkeypatch):
    # the (M,N,K) table chooses the kernel: a row naming a tile that cannot exist must surface as an error,
    # a valid row must be honoured, and an untuned shape must still run (heuristic)
    from aiter_b200 import gemm_op_a8w4
    from aiter_b200.config import get_cu_num, get_gfx

    csv = tmp_path / "a8w4.csv"
    csv.write_text(
        "gfx,cu_num,M,N,K,kernelId,splitK,us,kernelName,tflops,bw,errRatio\n"
        f"{get_gfx()},{get_cu_num()},32,512,1024,0,0,1.0,tc5_128x32_t_s4,0,0,0\n"
        f"{get_gfx()},{get_cu_num()},48,512,1024,0,0,1.0,tc5_128x999_t_s4,0,0,0\n")
    monkeypatch.setenv("AITER_CONFIG_GEMM_A8W4_MXFP8", str(csv))
    gemm_op_a8w4._table.clear()
    try:
        assert gemm_op_a8w4.get_A8W4_config(32, 512, 1024)["kernelName"] == "tc5_128x32_t_s4"
        assert gemm_op_a8w4.get_A8W4_config(17, 512, 1024)["kernelName"] == "tc5_128x32_t_s4"  # padded M (gl=0: 32)
        ref, args = a8w4_case(ab, 32, 512, 1024, 0, seed=17)
        check(ref, ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False), what="table row honoured")
        ref, args = a8w4_case(ab, 48, 512, 1024, 0, seed=18)
        with pytest.raises(RuntimeError, match="not find kernel"):
            ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False)
        ref, args = a8w4_case(ab, 100, 512, 1024, 0, seed=19)
        check(ref, ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False), what="untuned shape")
    finally:
        gemm_op_a8w4._table.clear()
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- fp8, fp32 128-block scales
@pytest.mark.parametrize("M,N,K,bpre", [(1, 128, 128, False), (48, 512, 1024, False), (48, 512, 1024, True), (300, 1024, 2048, True),
                                       (128, 4096, 4096, False), (130, 320, 640, True), (1024, 2048, 512, False),
                                       # more 128x128 tiles than SMs: the 256x256 CTA-pair kernel (ragged M and N)
                                       (640, 4096, 512, False), (1300, 2304, 640, True),
                                       # few rows (weights on the M side of the MMA), K split across CTAs, ragged N
                                       (16, 4096, 4096, False), (17, 1536, 7168, True), (33, 400, 2048, False), (64, 7168, 2048, True),
                                       (5, 128, 896, False), (100, 1024, 4096, False),
                                       # more K blocks per slice than TMEM partials and stages: both MMA issuers wrap their rings
                                       (8, 4096, 8192, False), (24, 2048, 16384, True)])
def test_a8w8_blockscale_fp32_scales(ab, M, N, K, bpre):
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, generator=g) + 0.25
    ws = torch.rand((N + 127) // 128, K // 128, generator=g) + 0.25
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), xs.numpy(), ws.numpy())
    if bpre:
        xs_t = xs.T.contiguous().cuda()  # K-block-major storage
        wq = ab.shuffle_weight(w.cuda(), layout=(16, 16))
        out = ab.gemm_a8w8_blockscale_bpreshuffle(x.cuda(), wq, xs_t.view(M, K // 128), ws.cuda())
        check(ref, out, what=f"blockscale bpreshuffle (re-viewed x_scale) {M}x{N}x{K}")
        out = ab.gemm_a8w8_blockscale_bpreshuffle(x.cuda(), wq, xs_t.T, ws.cuda())
        check(ref, out, what=f"blockscale bpreshuffle (strided x_scale) {M}x{N}x{K}")
    else:
        out = ab.gemm_a8w8_blockscale(x.cuda(), w.cuda(), xs.cuda(), ws.cuda())
        check(ref, out, what=f"blockscale {M}x{N}x{K}")
    assert_healthy(ab)


@pytest.mark.parametrize("M", [65, 128, 200, 256, 520, 1024])
def test_a8w8_blockscale_few_rows_kernel_on_several_tiles_of_64_rows(ab, M):
    # by name the few-rows kernel takes up to 1024 rows: every tile of 64 is a CTA of its own on the same weight tile;
    # unsplit, cluster K splits and fp16 output, fp32 and e8m0 scales, ragged N
    N, K = 400, 2048
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, generator=g) + 0.25
    ws = torch.rand((N + 127) // 128, K // 128, generator=g) + 0.25
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), xs.numpy(), ws.numpy())
    for name in ("bs_fewrows_k0", "bs_fewrows_k1", "bs_fewrows_k3"):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ab.gemm_a8w8_blockscale_cktile(x.cuda(), w.cuda(), xs.cuda(), ws.cuda(), out, kernelName=name)
        check(ref, out, what=f"blockscale {M} rows {name}")
    out16 = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    xs_t = xs.T.contiguous().cuda()  # the preshuffled form stores x_scale K-block-major
    ab.gemm_a8w8_blockscale_cktile(x.cuda(), ab.shuffle_weight(w.cuda(), layout=(16, 16)), xs_t.view(M, K // 128), ws.cuda(), out16,
                                   preshuffleB=True, kernelName="bs_fewrows_k2")
    got, want = out16.float().cpu().numpy(), ox.bf16_bits_to_f32(ref)
    assert np.all(np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want))
    exs = torch.randint(124, 130, (M, K // 128), generator=g, dtype=torch.uint8)
    ews = torch.randint(124, 130, ((N + 127) // 128, K // 128), generator=g, dtype=torch.uint8)
    ref8 = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), ox.e8m0_to_f32(exs.numpy()), ox.e8m0_to_f32(ews.numpy()))
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ab.gemm_a8w8_blockscale_cktile(x.cuda(), w.cuda(), exs.cuda().view(ab.dtypes.fp8_e8m0), ews.cuda().view(ab.dtypes.fp8_e8m0), out,
                                   kernelName="bs_fewrows_k1")
    check(ref8, out, what=f"blockscale {M} rows, e8m0 scales, bs_fewrows_k1")
    assert_healthy(ab)


@pytest.mark.parametrize("M,N,K", [(2500, 2320, 384), (300, 640, 1024), (4100, 4608, 128)])
def test_a8w8_blockscale_pair_kernels_by_name(ab, M, N, K):
    # the CTA-pair kernels: bs_256x256 is persistent (the first shape gives every pair more than one tile, with an odd
    # number of K blocks so that the TMEM partials change parity from tile to tile; the last one three tiles of one K
    # block each), bs_256x128 runs one tile per pair; ragged M and N, row-major and preshuffled weights, 16- and 32-bit outputs
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, generator=g) + 0.25
    ws = torch.rand((N + 127) // 128, K // 128, generator=g) + 0.25
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), xs.numpy(), ws.numpy())
    want = ox.bf16_bits_to_f32(ref)
    xc, wc, xsc, wsc = x.cuda(), w.cuda(), xs.cuda(), ws.cuda()
    wq, xs_t = ab.shuffle_weight(wc, layout=(16, 16)), xs.T.contiguous().cuda()
    for name in ("bs_256x256", "bs_256x128"):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        before = ab.launch_count()
        ab.gemm_a8w8_blockscale_cktile(xc, wc, xsc, wsc, out, kernelName=name)
        assert ab.launch_count() == before + 1
        check(ref, out, what=f"blockscale {M}x{N}x{K} {name}")
        out16 = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        ab.gemm_a8w8_blockscale_cktile(xc, wq, xs_t.view(M, K // 128), wsc, out16, preshuffleB=True, kernelName=name)
        got = out16.float().cpu().numpy()
        assert np.all(np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want)), f"{name} preshuffled, fp16 output"
        out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        ab.gemm_a8w8_blockscale_cktile(xc, wc, xsc, wsc, out32, kernelName=name)
        got = out32.cpu().numpy()
        assert np.all(np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want)), f"{name} fp32 output"
        # an output pitch that rules out tile stores (rows start on odd 2-byte offsets): plain stores
        wide = torch.full((M, N + 3), float("nan"), dtype=torch.bfloat16, device="cuda")
        ab.gemm_a8w8_blockscale_cktile(xc, wc, xsc, wsc, wide[:, :N], kernelName=name)
        check(ref, wide[:, :N], what=f"blockscale {M}x{N}x{K} {name}, strided output")
        assert torch.isnan(wide[:, N:]).all()
    assert_healthy(ab)


@pytest.mark.parametrize("M", [16, 100, 300])
def test_a8w8_blockscale_replays_from_a_cuda_graph(ab, M):
    # few-rows kernel (cluster + dependent launch), 128x128 kernel with and without its workspace K split: captured after
    # one call on the capture stream (the workspace may not grow during capture), replayed, compared with the oracle
    N, K = 1024, 2048
    g = torch.Generator().manual_seed(77 + M)
    x = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, generator=g) + 0.5
    ws = torch.rand(N // 128, K // 128, generator=g) + 0.5
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), xs.numpy(), ws.numpy())
    xc, wc, xsc, wsc = x.cuda(), w.cuda(), xs.cuda(), ws.cuda()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        ab.gemm_a8w8_blockscale_cktile(xc, wc, xsc, wsc, out)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(3):
                ab.gemm_a8w8_blockscale_cktile(xc, wc, xsc, wsc, out)
        out.fill_(float("nan"))
        graph.replay()
        graph.replay()
    torch.cuda.synchronize()
    check(ref, out, what=f"blockscale from a CUDA graph, M={M}")
    assert_healthy(ab)


def test_a8w8_blockscale_other_backend_names(ab):
    # the CK-tile and assembly names of the reference reach the same kernels, each in its own argument order
    M, N, K = 200, 512, 1024
    g = torch.Generator().manual_seed(31)
    x = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, generator=g) + 0.25
    ws = torch.rand(N // 128, K // 128, generator=g) + 0.25
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(), xs.numpy(), ws.numpy())
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    wq = ab.shuffle_weight(w.cuda(), layout=(16, 16))
    xs_t = xs.T.contiguous().cuda()
    check(ref, ab.flatmm_a8w8_blockscale_asm(x.cuda(), w.cuda(), xs.cuda(), ws.cuda(), out), what="flatmm_a8w8_blockscale_asm")
    out.zero_()
    check(ref, ab.gemm_a8w8_blockscale_cktile(x.cuda(), w.cuda(), xs.cuda(), ws.cuda(), out), what="gemm_a8w8_blockscale_cktile")
    out.zero_()
    check(ref, ab.gemm_a8w8_blockscale_bpreshuffle_cktile(x.cuda(), wq, xs_t.T, ws.cuda(), out), what="..._bpreshuffle_cktile")
    out.zero_()
    check(ref, ab.gemm_a8w8_blockscale_bpreshuffle_asm(x.cuda(), wq, out, xs_t.T, ws.cuda()), what="..._bpreshuffle_asm")
    with pytest.raises(RuntimeError, match="bias"):
        ab.gemm_a8w8_blockscale_bpreshuffle_asm(x.cuda(), wq, out, xs_t.T, ws.cuda(), bias=torch.zeros(N, device="cuda"))
    assert_healthy(ab)


@pytest.mark.parametrize("M,N,K,bpre", [(64, 256, 512, False), (300, 1024, 2048, True), (1, 128, 128, False),
                                       (16, 4096, 4096, False), (32, 1536, 7168, True), (7, 400, 1024, True),
                                       # shapes whose tuned-table row names an fp32-scale kernel (bs_128x128, bs_256x256)
                                       (128, 4096, 4096, False), (1024, 4096, 4096, True)])
def test_a8w8_blockscale_e8m0_scales_run_as_mxfp8(ab, M, N, K, bpre):
    # power-of-two scales ride the block-scaled MMA: two small expansion launches + the MXFP8 kernel; up to 64 rows
    # the few-rows blockscale kernel reads the e8m0 bytes itself
    g = torch.Generator().manual_seed(5 + M)
    x = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    xs = torch.randint(124, 130, (M, K // 128), generator=g, dtype=torch.uint8)
    ws = torch.randint(124, 130, ((N + 127) // 128, K // 128), generator=g, dtype=torch.uint8)
    ref = ox.gemm_a8w8_blockscale_ref(x.view(torch.uint8).numpy(), w.view(torch.uint8).numpy(),
                                      ox.e8m0_to_f32(xs.numpy()), ox.e8m0_to_f32(ws.numpy()))
    before = ab.launch_count()
    if bpre:
        xs_t = xs.T.contiguous().cuda()  # K-block-major storage
        out = ab.gemm_a8w8_blockscale_bpreshuffle(x.cuda(), ab.shuffle_weight(w.cuda(), layout=(16, 16)),
                                                  xs_t.T.view(ab.dtypes.fp8_e8m0), ws.cuda().view(ab.dtypes.fp8_e8m0))
    else:
        out = ab.gemm_a8w8_blockscale(x.cuda(), w.cuda(), xs.cuda().view(ab.dtypes.fp8_e8m0), ws.cuda().view(ab.dtypes.fp8_e8m0))
    # one launch where the few-rows kernel serves the call (up to 64 rows; up to 256 while its tiles of 64 rows all fit the
    # machine at once; or a tuned row that names it: it reads the e8m0 bytes itself), else two expansion launches + the
    # MXFP8 kernel
    from aiter_b200 import gemm_op_a8w8
    from aiter_b200.config import get_cu_num
    row = gemm_op_a8w8.get_CKGEMM_config(M, N, K, bpreshuffle=bpre)
    fits = M <= 256 and -(-N // 128) * -(-M // 64) <= get_cu_num()
    few = M <= 64 or fits or (row is not None and str(row.get("kernelName") or "").startswith("bs_fewrows"))
    assert ab.launch_count() == before + (1 if few else 3)
    check(ref, out, what=f"blockscale with e8m0 scales {M}x{N}x{K} bpre={bpre}")
    # one e8m0 and one fp32 scale tensor: the e8m0 one is widened, the fp32 kernel runs
    out = ab.gemm_a8w8_blockscale(x.cuda(), w.cuda(), xs.cuda().view(ab.dtypes.fp8_e8m0), ab.fp4_utils.e8m0_to_f32(ws.cuda()))
    check(ref, out, what="blockscale with mixed scale dtypes")
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- decode kernel, several activation tiles
@pytest.mark.parametrize("M", [65, 128, 200, 256])
def test_decode_kernel_on_up_to_four_tiles_of_64_rows(ab, M):
    # a 128x64 or 128x128 tile with the weights on the 128-row slot and a K split of at most 4 runs on the decode kernel;
    # with more activation rows than the tile is wide every tile is a CTA of its own on the same weight tile (ragged last
    # tile included); a 128-column tile leaves the epilogue in two chunks of 64 columns
    N, K = 640, 1024
    for name in ("tc5_128x64_t_s0_k0", "tc5_128x64_t_s3_k1", "tc5_128x64_t_s0_k2", "tc5_128x128_t_s0_k0", "tc5_128x128_t_s2_k1"):
        apre = 1 if M % 2 == 0 else 0  # the (m/2,k/128,2,128) activation tiling needs an even row count
        ref, args = mxfp8_case(ab, M, N, K, apre, seed=M)
        check(ref, ab.gemm_a8w8_mxfp8(*args, a_preshuffle=bool(apre), kernelName=name), what=f"mxfp8 {M} rows {name}")
        ref, args = a8w4_case(ab, M, N, K, 0, seed=M + 1)
        check(ref, ab.gemm_a8w4_mxfp8(*args, a_preshuffle=False, kernelName=name), what=f"a8w4 {M} rows {name}")
        ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K, seed=M + 2)
        out = torch.full(((M + 31) // 32 * 32, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ab.gemm_a4w4_asm(to_cuda_u8(xq, ab.dtypes.fp4x2), ab.shuffle_weight(to_cuda_u8(wq), layout=(16, 16)),
                         ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws)), out, name)
        check(ref, out[:M], what=f"mxfp4 {M} rows {name}")
        assert torch.isnan(out[M:].float()).all(), "rows beyond M must stay untouched"
        a, b = randn_bf16(M, K, M + 3, 0.1), randn_bf16(N, K, M + 4, 0.1)
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ab.gemm_a16w16_asm(a.cuda(), b.cuda(), y, kernelName=name)
        check(ox.gemm_a16w16_ref(bf16_bits(a), bf16_bits(b)), y, what=f"bf16 {M} rows {name}")
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- persistent paths
def test_many_units_per_cta(ab):
    # more output tiles than SMs: the persistent loop, both accumulators and the stage ring wrap many times
    M, N, K = 2048, 4096, 512
    ref, args = mxfp8_case(ab, M, N, K, 0, seed=21)
    for name in ("tc5_128x64_n_s3", "tc5_256x128_n_s4", "tc5_256x256_n_s5", ""):
        out = ab.gemm_a8w8_mxfp8(*args, a_preshuffle=False, kernelName=name)
        check(ref, out, what=f"mxfp8 {M}x{N}x{K} {name or 'heuristic'}")
    assert_healthy(ab)
    a = randn_bf16(M, K, 31, 0.1)
    b = randn_bf16(N, K, 32, 0.1)
    refb = ox.gemm_a16w16_ref(bf16_bits(a), bf16_bits(b))
    for kid in (22, 1034, 1043):
        y = torch.full((1, M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ab.opus_gemm_a16w16_tune(a.cuda()[None], b.cuda()[None], y, None, kid, 0)
        check(refb, y[0], what=f"bf16 kernelId {kid}")
    assert_healthy(ab)


def test_mxfp4_large_pair_tiles(ab):
    # M >= 1024, K >= 4096 and K % 256 == 0: both e8m0_shuffle scale tensors are re-laid once (two extra launches)
    M, N, K = 1024, 1792, 4096
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K, seed=23)
    args = (to_cuda_u8(xq, ab.dtypes.fp4x2), ab.shuffle_weight(to_cuda_u8(wq)),
            ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws)))
    before = ab.launch_count()
    out = ab.gemm_a4w4(*args)
    assert ab.launch_count() == before + 3
    check(ref, out, what="gemm_a4w4 1024x1792x4096 (heuristic)")
    check(ref, ab.gemm_a4w4(*args), what="gemm_a4w4 1024x1792x4096, second call")
    assert_healthy(ab)


def test_mxfp4_tall_ragged_keeps_the_in_kernel_scale_path(ab):
    # K % 256 != 0: no re-layout pass, the e8m0_shuffle order is consumed by the kernel itself
    M, N, K = 1100, 512, 1216
    ref, xq, wq, xs, ws = mxfp4_case(ab, M, N, K, seed=25)
    before = ab.launch_count()
    out = ab.gemm_a4w4(to_cuda_u8(xq, ab.dtypes.fp4x2), ab.shuffle_weight(to_cuda_u8(wq)),
                       ab.fp4_utils.e8m0_shuffle(to_cuda_u8(xs)), ab.fp4_utils.e8m0_shuffle(to_cuda_u8(ws)))
    assert ab.launch_count() == before + 1
    check(ref, out, what="gemm_a4w4 1100x512x1216")
    assert_healthy(ab)


# ------------------------------------------------------------------------------------------- errors
def test_errors_are_python_exceptions(ab):
    a = torch.zeros((4, 100), dtype=torch.float8_e4m3fn, device="cuda")
    b = torch.zeros((16, 100), dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.zeros((32, 4), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="K must be divisible by 128"):
        ab.gemm_a8w8_mxfp8(a, b, s, s, a_preshuffle=False)
    with pytest.raises(RuntimeError, match="not find kernel"):
        x = torch.zeros((4, 128), dtype=torch.float8_e4m3fn, device="cuda")
        w = torch.zeros((16, 128), dtype=torch.float8_e4m3fn, device="cuda")
        ab.gemm_a8w8_mxfp8(x, w, s, s, a_preshuffle=False, kernelName="no_such_kernel")
    assert_healthy(ab)


def test_torch_ops_namespace_runs_the_cuda_path(ab):
    M, N, K = 64, 256, 512
    g = torch.Generator().manual_seed(11)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    xq, xs = ox.quant_mxfp4(x.float().numpy())
    wq, ws = ox.quant_mxfp4(w.float().numpy())
    ref = ox.gemm_a4w4_ref(xq, wq, xs, ws)
    before = ab.launch_count()
    out = torch.ops.aiter.gemm_a4w4(torch.from_numpy(xq).cuda(), ab.shuffle_weight(torch.from_numpy(wq).cuda(), layout=(16, 16)),
                                    ab.shuffle_scale(torch.from_numpy(xs).cuda()), ab.shuffle_scale(torch.from_numpy(ws).cuda()))
    assert ab.launch_count() == before + 1
    check(ref, out, what="torch.ops.aiter.gemm_a4w4")


def test_empty_activation_batch_is_a_no_op(ab):
    # M = 0: every operator returns an empty [0, N] tensor and launches nothing
    N, K = 256, 512
    before = ab.launch_count()
    w8 = ab.shuffle_mxfp8fp4_b(torch.zeros(N, K, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn))
    s_w = ab.shuffle_mxfp8fp4_scale(torch.full((N, K // 32), 0x7F, dtype=torch.uint8, device="cuda"))
    s_a = torch.empty(0, K // 32, dtype=torch.uint8, device="cuda")
    out = ab.gemm_a8w8_mxfp8(torch.empty(0, K, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn), w8, s_a, s_w, a_preshuffle=False)
    assert out.shape == (0, N)
    out = ab.tgemm.mm(torch.empty(0, K, dtype=torch.bfloat16, device="cuda"), torch.zeros(N, K, dtype=torch.bfloat16, device="cuda"))
    assert out.shape == (0, N)
    assert ab.launch_count() == before
    assert_healthy(ab)
