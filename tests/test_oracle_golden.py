"""The numpy oracle against vectors produced by the reference's own functions."""
import numpy as np

from oracle import mx_oracle as ox


def test_e2m1_known_answers(golden):
    assert np.array_equal(ox.f32_to_e2m1(golden["e2m1_probe_in"]), golden["e2m1_probe_out"])
    # the facts the reference documents: ties to even code, saturation, sign kept on zero
    probe = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 100.0, -7.0, -0.0, -0.1, 0.2500001], dtype=np.float32)
    assert ox.f32_to_e2m1(probe).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 7, 0xF, 8, 8, 1]


def test_e2m1_lut(golden):
    allb = np.arange(256, dtype=np.uint8).reshape(-1, 1)
    assert np.array_equal(ox.e2m1_to_f32(allb).view(np.uint32), golden["e2m1_lut"].view(np.uint32))


def test_e8m0_scale(golden):
    amax = golden["amax_in"]
    assert np.array_equal(ox.e8m0_scale_roundup(amax, 6.0), golden["amax_e8m0_fp4"])
    assert np.array_equal(ox.e8m0_scale_roundup(amax, 448.0), golden["amax_e8m0_fp8"])
    # exact powers do not bump
    assert ox.e8m0_scale_roundup(np.float32([6.0, 12.0]), 6.0).tolist() == [127, 128]
    assert np.array_equal(ox.e8m0_to_f32(np.arange(256, dtype=np.uint8)).view(np.uint32), golden["e8m0_to_f32_bits"])


def test_e4m3_cast(golden):
    assert np.array_equal(ox.f32_to_e4m3fn(golden["e4m3_in"]), golden["e4m3_out"])
    dec = ox.e4m3fn_to_f32(np.arange(256, dtype=np.uint8))
    ref = golden["e4m3_decode_bits"].view(np.float32)
    ok = (dec == ref) | (np.isnan(dec) & np.isnan(ref))
    assert ok.all()
    fin = ~np.isnan(ref)
    assert np.array_equal(np.signbit(dec[fin]), np.signbit(ref[fin]))


def test_block_quantisers_bit_exact(golden):
    x = ox.bf16_bits_to_f32(golden["quant_in_bf16"])
    q4, s4 = ox.quant_mxfp4(x)
    assert np.array_equal(q4, golden["quant_fp4_data"])
    assert np.array_equal(s4, golden["quant_fp4_scale"])
    assert s4[0, 0] == 0 and (q4[0, :16] == 0).all()  # all-zero block: byte 0, nibbles 0
    q8, s8 = ox.quant_mxfp8(x)
    assert np.array_equal(q8, golden["quant_fp8_data"])
    assert np.array_equal(s8, golden["quant_fp8_scale"])


def test_shuffles(golden):
    assert np.array_equal(ox.shuffle_weight_16x16(golden["shufw_u8_in"]), golden["shufw_u8_out"])
    assert np.array_equal(ox.shuffle_weight_16x16(golden["shufw_i16_in"]), golden["shufw_i16_out"])
    assert np.array_equal(ox.e8m0_shuffle(golden["shufs_in"]), golden["shufs_out"])
    assert np.array_equal(ox.shuffle_mxfp8fp4_a(golden["g1250_a_in"]), golden["g1250_a_out"])
    assert np.array_equal(ox.shuffle_mxfp8fp4_b(golden["g1250_b_in"]), golden["g1250_b_out"])
    assert np.array_equal(ox.shuffle_mxfp8fp4_scale(golden["g1250_s_in"]), golden["g1250_s_out"])
    # for 1-byte elements the (16,16) weight shuffle and the 16x16 tile transpose coincide
    assert np.array_equal(golden["shufw_u8_out"], golden["g1250_b_out"])


def test_shuffle_index_formulas(golden):
    w = golden["shufw_u8_in"]
    flat = golden["shufw_u8_out"].reshape(-1)
    n_idx, k_idx = np.meshgrid(np.arange(w.shape[0]), np.arange(w.shape[1]), indexing="ij")
    assert np.array_equal(flat[ox.tile16_offset(n_idx, k_idx, w.shape[1])], w)
    s = golden["shufs_ragged_in"]
    out = golden["shufs_ragged_out"]
    m_idx, k_idx = np.meshgrid(np.arange(s.shape[0]), np.arange(s.shape[1]), indexing="ij")
    assert out.shape == (256, 16)
    assert np.array_equal(out.reshape(-1)[ox.e8m0_shuffle_offset(m_idx, k_idx, out.shape[1])], s)


def test_gemm_references(golden):
    out = ox.gemm_a16w16_ref(golden["gemm_bf16_a"], golden["gemm_bf16_b"])
    assert ox.mismatch_ratio(golden["gemm_bf16_out"], out, 1e-2, 1e-2) == 0.0
    out = ox.gemm_a4w4_ref(golden["gemm_a4w4_x"], golden["gemm_a4w4_w"], golden["gemm_a4w4_xs"], golden["gemm_a4w4_ws"])
    assert ox.mismatch_ratio(golden["gemm_a4w4_out"], out, 1e-2, 1e-2) == 0.0
    out = ox.gemm_a8w8_mxfp8_ref(golden["gemm_a8w8_x"], golden["gemm_a8w8_w"], golden["gemm_a8w8_xs"], golden["gemm_a8w8_ws"])
    assert ox.mismatch_ratio(golden["gemm_a8w8_out"], out, 1e-2, 1e-2) == 0.0
    out = ox.gemm_a8w4_mxfp8_ref(golden["gemm_a8w8_x"], golden["gemm_a4w4_w"], golden["gemm_a8w8_xs"], golden["gemm_a4w4_ws"])
    assert ox.mismatch_ratio(golden["gemm_a8w4_out"], out, 1e-2, 1e-2) == 0.0


def test_blockscale_reference(golden):
    out = ox.gemm_a8w8_blockscale_ref(golden["bs_x"], golden["bs_w"], golden["bs_xs"], golden["bs_ws"])
    assert ox.mismatch_ratio(golden["bs_out"], out, 1e-2, 1e-2) == 0.0
    out = ox.gemm_a8w8_blockscale_ref(golden["bs_x"], golden["bs_w"], ox.e8m0_to_f32(golden["bs_xs_e8m0"]), ox.e8m0_to_f32(golden["bs_ws_e8m0"]))
    assert ox.mismatch_ratio(golden["bs_out_e8m0"], out, 1e-2, 1e-2) == 0.0


def test_requantising_outputs_bit_exact(golden):
    y = golden["requant_in"]
    q8, s8 = ox.requant_mxfp8_blockN(y)
    assert np.array_equal(s8, golden["requant_fp8_scale"])
    assert np.array_equal(q8, golden["requant_fp8_data"])
    assert s8[0, 0] == 1 and s8[1, 0] == 127  # all-zero block -> byte 1 (amax clamped to FLT_MIN); amax 448 -> 2^0
    packed = ox.pack_mxfp8_out_scale(s8)
    assert np.array_equal(packed, golden["requant_fp8_scale_packed"])
    assert np.array_equal(ox.unpack_mxfp8_out_scale(packed, *y.shape), s8)
    assert np.array_equal(ox.requant_fp4(y), golden["requant_fp4_data"])


def test_nvfp4_reference(golden):
    ga, gb = golden["nv_g"]
    args = (golden["nv_x"], golden["nv_w"], golden["nv_xs"], golden["nv_ws"], ga, gb)
    y = ox.gemm_nvfp4_f32(*args)
    assert np.allclose(y, golden["nv_out_f32"], rtol=1e-5, atol=1e-4)  # fp32 sums in a different order
    assert ox.mismatch_ratio(golden["nv_out_bf16"], ox.gemm_nvfp4_ref(*args), 1e-2, 1e-2) == 0.0
    assert np.allclose(ox.gemm_nvfp4_f32(*args, noscale=True), golden["nv_out_noscale_f32"], rtol=1e-5, atol=1e-3)
    # the constant case of the reference's F4GEMM test (op_tests/test_f4gemm.py:169-178): A = 0x22 (1.0), B = 0x33 (1.5),
    # e4m3 scales 0x38 (1.0): every output is 1.5 * K
    k = 256
    a = np.full((4, k // 2), 0x22, dtype=np.uint8)
    b = np.full((8, k // 2), 0x33, dtype=np.uint8)
    one = lambda rows: np.full((rows, k // 16), 0x38, dtype=np.uint8)
    assert (ox.gemm_nvfp4_f32(a, b, one(4), one(8)) == 1.5 * k).all()
    assert (ox.gemm_nvfp4_f32(a, b, one(4), one(8), 0.5, 4.0) == 3.0 * k).all()


def test_constant_input_known_answer():
    # A = B = 0.5 with unit scales: every output is 0.25*K (op_tests/test_mxfp8fp4gemm.py:75-98)
    k = 256
    a = np.full((4, k), 0x30, dtype=np.uint8)  # e4m3 0.5
    s = np.full((4, k // 32), 0x7F, dtype=np.uint8)
    out = ox.bf16_bits_to_f32(ox.gemm_a8w8_mxfp8_ref(a, a, s, s))
    assert (out == 0.25 * k).all()
    b4 = np.full((4, k // 2), 0x11, dtype=np.uint8)  # e2m1 0.5 in both nibbles
    out = ox.bf16_bits_to_f32(ox.gemm_a8w4_mxfp8_ref(a, b4, s, s))
    assert (out == 0.25 * k).all()


def test_padded_m():
    assert [ox.get_padded_m(m, 4096, 4096, 0) for m in (1, 16, 17, 256, 257, 1024, 1025, 4096, 4097)] == [16, 16, 32, 256, 288, 1024, 1088, 4096, 4224]
    assert [ox.get_padded_m(m, 4096, 4096, 1) for m in (1, 2, 3, 17, 8193)] == [1, 2, 4, 32, 16384]
    assert ox.get_padded_m(8193, 4097, 128, 1) == 8192


def test_torch_form_of_the_oracle(golden):
    import torch

    from oracle import torch_ref as tr

    def t(name):
        return torch.from_numpy(golden[name].copy())

    def bits(x):
        return x.view(torch.int16).numpy().view(np.uint16)

    out = tr.gemm_a8w8_mxfp8(t("gemm_a8w8_x"), t("gemm_a8w8_w"), t("gemm_a8w8_xs"), t("gemm_a8w8_ws"))
    assert ox.mismatch_ratio(golden["gemm_a8w8_out"], bits(out)) == 0.0
    out = tr.gemm_a4w4(t("gemm_a4w4_x"), t("gemm_a4w4_w"), t("gemm_a4w4_xs"), t("gemm_a4w4_ws"))
    assert ox.mismatch_ratio(golden["gemm_a4w4_out"], bits(out)) == 0.0
    out = tr.gemm_a8w4_mxfp8(t("gemm_a8w8_x"), t("gemm_a4w4_w"), t("gemm_a8w8_xs"), t("gemm_a4w4_ws"))
    assert ox.mismatch_ratio(golden["gemm_a8w4_out"], bits(out)) == 0.0
    a = torch.from_numpy(golden["gemm_bf16_a"].view(np.int16).copy()).view(torch.bfloat16)
    b = torch.from_numpy(golden["gemm_bf16_b"].view(np.int16).copy()).view(torch.bfloat16)
    assert ox.mismatch_ratio(golden["gemm_bf16_out"], bits(tr.gemm_a16w16(a, b))) == 0.0
