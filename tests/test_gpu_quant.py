"""Fused 1x32 MX quantiser (CUDA) against the oracle: data bytes, scale bytes and scale layouts are bit-exact."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as ox

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def bf16_input(M, K, seed, kind="randn"):
    g = torch.Generator().manual_seed(seed)
    if kind == "randn":
        x = torch.randn(M, K, generator=g) * torch.exp2(torch.randint(-12, 12, (M, 1), generator=g).float())
    elif kind == "edges":
        # zeros, +-0, huge, tiny, exact ties of the e2m1 grid after scaling, and a negative constant block
        vals = torch.tensor([0.0, -0.0, 1e4, 1e-10, -3.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 448.0, 449.0, 12.0, -0.1])
        x = vals[torch.randint(0, len(vals), (M, K), generator=g)]
        x[0, :32] = 0.0
        x[M - 1, -32:] = -3.0
    return x.to(torch.bfloat16)


def unshuffle_e8m0(s, M, KB):
    s = s.view(torch.uint8).cpu().numpy()
    mm, kk = np.meshgrid(np.arange(M), np.arange(KB), indexing="ij")
    return s.reshape(-1)[ox.e8m0_shuffle_offset(mm, kk, s.shape[1])]


# (2080 x 8192 is more than 2048 tiles: the warp-per-tile kernel; the others run one CTA per tile)
@pytest.mark.parametrize("M,K", [(1, 32), (33, 320), (300, 1024), (256, 4096), (17, 7168), (2080, 8192)])
@pytest.mark.parametrize("kind", ["randn", "edges"])
def test_quant_mxfp4_bit_exact(ab, M, K, kind):
    x = bf16_input(M, K, seed=M + K, kind=kind)
    ref_q, ref_s = ox.quant_mxfp4(x.float().numpy())
    for shuffle in (False, True):
        y, s = ab.per_1x32_mx_quant_hip(x.cuda(), quant_dtype=ab.dtypes.fp4x2, shuffle=shuffle)
        assert y.shape == (M, K // 2)
        assert np.array_equal(y.view(torch.uint8).cpu().numpy(), ref_q), f"packed e2m1 differs (shuffle={shuffle})"
        if shuffle:
            assert s.shape == ((M + 255) // 256 * 256, (K // 32 + 7) // 8 * 8)
            got = unshuffle_e8m0(s, M, K // 32)
        else:
            assert s.shape == (M, K // 32)
            got = s.view(torch.uint8).cpu().numpy()
        assert np.array_equal(got, ref_s), f"scale bytes differ (shuffle={shuffle})"


@pytest.mark.parametrize("M,K", [(1, 128), (33, 384), (300, 1024), (64, 4096), (4100, 4096)])
@pytest.mark.parametrize("kind", ["randn", "edges"])
def test_quant_mxfp8_bit_exact(ab, M, K, kind):
    x = bf16_input(M, K, seed=7 * M + K, kind=kind)
    ref_q, ref_s = ox.quant_mxfp8(x.float().numpy())
    y, s = ab.per_1x32_mx_quant_hip(x.cuda(), quant_dtype=ab.dtypes.fp8, scale_type=ab.dtypes.fp8_e8m0, shuffle=False)
    assert np.array_equal(y.view(torch.uint8).cpu().numpy(), ref_q)
    assert np.array_equal(s.view(torch.uint8).cpu().numpy(), ref_s)
    # the MXFP8 GEMM's own scale order: identical to shuffling the plain scales on the host
    y2, s2 = ab.per_1x32_mx_quant_hip(x.cuda(), quant_dtype=ab.dtypes.fp8, scale_type=ab.dtypes.fp8_e8m0, shuffle=2)
    assert np.array_equal(y2.view(torch.uint8).cpu().numpy(), ref_q)
    want = ab.shuffle_mxfp8fp4_scale(torch.from_numpy(ref_s).cuda())
    assert torch.equal(s2.view(torch.uint8).reshape(-1), want.view(torch.uint8).reshape(-1))


def test_quantise_then_gemm_matches_oracle(ab):
    # the serving sequence: activations quantised on the GPU straight into the GEMM's scale layout
    M, N, K = 96, 512, 1024
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    xq, xs = ox.quant_mxfp4(x.float().numpy())
    wq, ws = ox.quant_mxfp4(w.float().numpy())
    ref = ox.gemm_a4w4_ref(xq, wq, xs, ws)
    a, sa = ab.per_1x32_mx_quant_hip(x.cuda(), quant_dtype=ab.dtypes.fp4x2, shuffle=True)
    b, sb = ab.per_1x32_mx_quant_hip(w.cuda(), quant_dtype=ab.dtypes.fp4x2, shuffle=True)
    out = ab.gemm_a4w4(a, ab.shuffle_weight(b.view(torch.uint8), layout=(16, 16)), sa, sb)
    from helpers import check

    check(ref, out, what="per_1x32_mx_quant_hip -> gemm_a4w4")


def test_quant_rejects_what_is_not_built(ab):
    x = torch.randn(4, 64).to(torch.bfloat16).cuda()
    with pytest.raises(NotImplementedError):
        ab.per_1x32_mx_quant_hip(x, quant_dtype=ab.dtypes.fp8)
    with pytest.raises(RuntimeError, match="group_size"):
        ab.dynamic_per_group_scaled_quant(torch.empty(4, 32, dtype=torch.uint8, device="cuda"), x,
                                          torch.empty(4, 2, dtype=torch.uint8, device="cuda"), 64, False)


def test_torch_quantisers_give_the_same_bytes_on_cpu_and_gpu(ab):
    """The full-size parity tests and bench.py quantise on the GPU with the torch path and check against a CPU oracle:
    that is only sound if the torch path produces the same bytes on both devices (elementwise bit operations,
    divisions by powers of two and dtype casts).  300 x 1024 with every edge case of the quantiser tests."""
    x = bf16_input(300, 1024, seed=7, kind="edges")
    x[10:200] = bf16_input(190, 1024, seed=8, kind="randn")
    for fn, kw in ((ab.per_1x32_f4_quant, {}), (ab.per_1x32_f8_scale_f8_quant, {"scale_type": ab.dtypes.fp8_e8m0})):
        q_cpu, s_cpu = fn(x, **kw)
        q_gpu, s_gpu = fn(x.cuda(), **kw)
        assert torch.equal(q_cpu.view(torch.uint8), q_gpu.view(torch.uint8).cpu()), f"{fn.__name__}: data bytes differ between cpu and cuda"
        assert torch.equal(s_cpu.view(torch.uint8), s_gpu.view(torch.uint8).cpu()), f"{fn.__name__}: scale bytes differ between cpu and cuda"
    # and the oracle agrees with both (the CPU tests pin this on the golden vectors; here on this tensor)
    q4, s4 = ox.quant_mxfp4(x.float().numpy())
    q, s = ab.per_1x32_f4_quant(x.cuda())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), q4) and np.array_equal(s.view(torch.uint8).cpu().numpy(), s4)
    q8, s8 = ox.quant_mxfp8(x.float().numpy())
    q, s = ab.per_1x32_f8_scale_f8_quant(x.cuda(), scale_type=ab.dtypes.fp8_e8m0)
    ok = np.array_equal(q.view(torch.uint8).cpu().numpy(), q8) and np.array_equal(s.view(torch.uint8).cpu().numpy(), s8)
    assert ok
