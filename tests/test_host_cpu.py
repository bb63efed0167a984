"""Host-side logic that needs no GPU: the library loads and exports every declared symbol, the torch
host functions reproduce the reference-generated golden vectors bit for bit, errors cross the C ABI as
RuntimeError, and the tuned-table look-up follows the reference's rules."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def test_library_exports_every_declared_symbol(ab):
    header = open(os.path.join(ROOT, "include", "aiter_b200.h")).read()
    declared = re.findall(r"AITER_B200_API\s+[\w\s\*]+?\b(\w+)\s*\(", header)
    assert len(declared) >= 18, declared
    lib = ctypes.CDLL(ab._ffi.LIB_PATH)
    missing = [name for name in declared if not hasattr(lib, name)]
    assert not missing, f"declared in include/aiter_b200.h but not exported: {missing}"
    assert lib.aiter_ctypes_abi_version() == 2
    assert set(ab._ffi.SIGNATURES) <= set(declared)


def test_struct_layout_matches_header(ab):
    assert ctypes.sizeof(ab._ffi.aiter_tensor_t) == 160
    t = ab._ffi.torch_to_aiter(torch.zeros(3, 5, dtype=torch.bfloat16)[:, 1:4])
    assert (t.ndim, t.shape[0], t.shape[1], t.strides[0], t.strides[1], t.dtype_, t.device_id) == (2, 3, 3, 5, 1, 3, -1)
    assert ab.dtypes.aiter_dtype_id(torch.uint8) == 11 and ab.dtypes.aiter_dtype_id(ab.dtypes.fp4x2) == 6


def test_padded_m_matches_oracle(ab):
    from oracle import mx_oracle as ox

    for m in (1, 15, 16, 17, 255, 256, 257, 1000, 1024, 1025, 4095, 4097, 8191, 8193, 20000):
        for n in (1024, 4096, 8192):
            for gl in (0, 1):
                assert ab.get_padded_m(m, n, 4096, gl) == ox.get_padded_m(m, n, 4096, gl), (m, n, gl)


def test_errors_cross_the_abi_as_runtime_error(ab):
    a = torch.zeros((4, 128), dtype=torch.float8_e4m3fn)
    s = torch.zeros((32, 4), dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="mxfp8_mxfp8_gemm_asm failed: .*must live on a GPU"):
        ab.gemm_a8w8_mxfp8(a, a, s, s, a_preshuffle=False)  # CPU tensors are refused before any launch
    with pytest.raises(RuntimeError, match="opus_gemm_a16w16_tune failed: .*XQ must live on a GPU"):
        x = torch.zeros((1, 4, 64), dtype=torch.bfloat16)
        ab.opus_gemm_a16w16_tune(x, x, torch.zeros((1, 4, 4), dtype=torch.bfloat16), None, 999, 0)
    with pytest.raises(ValueError, match="must be 3D"):
        ab.opus_gemm_a16w16_tune(torch.zeros(4, 64), torch.zeros(4, 64), torch.zeros(4, 4))
    # an out-of-range K split is refused before it can reach a shift (log2 of the split: 0..8, -1 = library's choice)
    p4 = torch.zeros((32, 64), dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="gemm_a4w4_asm failed: .*K split must be between 0 and 8"):
        ab.gemm_a4w4_asm(p4, p4, s, s, torch.zeros((32, 32), dtype=torch.bfloat16), log2_k_split=40)
    with pytest.raises(RuntimeError, match="aiter_b200_gemm_a8w8_mxfp8_noalloc failed: .*must live on a GPU"):
        ab.gemm_a8w8_mxfp8_noalloc(a, a, s, s, torch.zeros((4, 4), dtype=torch.bfloat16), a_preshuffle=False)


def test_heuristic_and_kernel_menu(ab):
    name, l2 = ab.heuristic_name(1, 8192, 4096, 4096)
    assert name.startswith("tc5_256x") and l2 == 0  # tall problems run on CTA pairs
    name, l2 = ab.heuristic_name(2, 1, 7168, 16384)
    assert "_t_" in name and l2 >= 1  # decode shapes: weights on the 128-row slot, K split
    assert "kernelId" in ab.kernel_list()


def test_heuristic_follows_the_tuned_choices_it_was_fitted_to(ab):
    """choose_config on shapes of the reference's model list (MXFP4 = kind 2; 148 SMs assumed when no GPU is present):
    the tile family and K split the tuner picked for them on B200."""
    import re

    def pick(kind, M, N, K):
        name, l2 = ab.heuristic_name(kind, M, N, K)
        return re.sub(r"_s\d+$", "", name), l2

    # tall problems: CTA pairs; 192 columns (two accumulators) where the scales are re-laid and K is short, 256 at long K
    assert pick(2, 16384, 7168, 2048) == ("tc5_256x192_n", 0)
    assert pick(2, 16384, 7168, 16384) == ("tc5_256x256_n", 0)
    assert pick(2, 4096, 24576, 1536) == ("tc5_256x192_n", 0)   # tall by M x N
    assert pick(2, 4096, 7168, 2048) == ("tc5_256x256_n", 0)    # not tall: the scale warps set the pace, waves decide
    assert pick(4, 16384, 7168, 2048) == ("tc5_256x192_n", 0)   # NVFP4: its wire order is the cheap one
    # pairs from two dozen 256 x 256 tiles on, never split; below that single CTAs on the largest tile that fills half the machine
    assert pick(2, 512, 7168, 2048) == ("tc5_256x256_n", 0)
    assert pick(1, 1024, 4096, 4096) == ("tc5_256x256_n", 0)
    assert pick(2, 512, 2048, 6144) == ("tc5_128x64_n", 0)
    assert pick(2, 1024, 512, 4096) == ("tc5_128x64_n", 0)      # (a workspace split needs slices of 24 K tiles)
    # 65..256 rows: decode tiles of 64 rows while they fit the machine, of 128 rows for a large weight or when only those fit
    assert pick(2, 256, 7168, 2048) == ("tc5_128x64_t", 0)
    assert pick(2, 128, 4096, 4096) == ("tc5_128x64_t", 1)
    assert pick(2, 128, 7168, 16384) == ("tc5_128x128_t", 1)
    assert pick(2, 256, 16384, 4096) == ("tc5_128x128_t", 0)
    # clusters of four may take 7/8 of the two-CTAs-per-SM capacity: 72 weight tiles split two ways, not four
    assert pick(2, 64, 9216, 16384) == ("tc5_128x64_t", 1)
    assert pick(2, 16, 7168, 16384) == ("tc5_128x16_t", 2)


def test_host_numerics_against_golden(ab, golden):
    x = torch.from_numpy(golden["quant_in_bf16"].view(np.int16).copy()).view(torch.bfloat16)
    q4, s4 = ab.per_1x32_f4_quant(x)
    assert np.array_equal(q4.view(torch.uint8).numpy(), golden["quant_fp4_data"])
    assert np.array_equal(s4.view(torch.uint8).numpy(), golden["quant_fp4_scale"])
    q8, s8 = ab.per_1x32_f8_scale_f8_quant(x, scale_type=ab.dtypes.fp8_e8m0)
    assert np.array_equal(q8.view(torch.uint8).numpy(), golden["quant_fp8_data"])
    assert np.array_equal(s8.view(torch.uint8).numpy(), golden["quant_fp8_scale"])
    assert np.array_equal(ab.fp4_utils.f32_to_e2m1_code(torch.from_numpy(golden["e2m1_probe_in"])).numpy(), golden["e2m1_probe_out"])
    amax = torch.from_numpy(golden["amax_in"])
    assert np.array_equal(ab.fp4_utils.f32_to_mx_e8m0_scale(amax, dtype=ab.MxDtype.FP4_E2M1).view(torch.uint8).numpy(), golden["amax_e8m0_fp4"])
    assert np.array_equal(ab.fp4_utils.f32_to_mx_e8m0_scale(amax, dtype=ab.MxDtype.FP8_E4M3).view(torch.uint8).numpy(), golden["amax_e8m0_fp8"])
    assert np.array_equal(ab.fp4_utils.mxfp4_to_f32(torch.arange(256, dtype=torch.uint8).view(-1, 1)).numpy().view(np.uint32),
                          golden["e2m1_lut"].view(np.uint32))
    assert ab.get_torch_quant(ab.QuantType.per_1x32) is ab.per_1x32_f4_quant


def test_shuffles_against_golden(ab, golden):
    t = torch.from_numpy
    w = ab.shuffle_weight(t(golden["shufw_u8_in"]))
    assert w.is_shuffled and np.array_equal(w.numpy(), golden["shufw_u8_out"])
    assert np.array_equal(ab.shuffle_weight(t(golden["shufw_i16_in"])).numpy(), golden["shufw_i16_out"])
    assert np.array_equal(ab.shuffle_scale(t(golden["shufs_in"])).numpy(), golden["shufs_out"])
    ragged = ab.shuffle_scale(t(golden["shufs_ragged_in"])).numpy()
    src = golden["shufs_ragged_in"]
    from oracle import mx_oracle as ox

    mm, kk = np.meshgrid(np.arange(src.shape[0]), np.arange(src.shape[1]), indexing="ij")
    assert np.array_equal(ragged.reshape(-1)[ox.e8m0_shuffle_offset(mm, kk, ragged.shape[1])], src)  # valid slots
    assert np.array_equal(ab.shuffle_mxfp8fp4_a(t(golden["g1250_a_in"])).numpy(), golden["g1250_a_out"])
    assert np.array_equal(ab.shuffle_mxfp8fp4_b(t(golden["g1250_b_in"])).numpy(), golden["g1250_b_out"])
    assert np.array_equal(ab.shuffle_mxfp8fp4_scale(t(golden["g1250_s_in"])).numpy(), golden["g1250_s_out"])
    with pytest.raises(AssertionError):
        ab.shuffle_weight(torch.zeros(8, 64, dtype=torch.uint8))  # N not a multiple of 16


def _write_csv(path, rows, header="gfx,cu_num,M,N,K,kernelId,splitK,us,kernelName,tflops,bw,errRatio"):
    path.write_text(header + "\n" + "\n".join(rows) + "\n")


def test_f4gemm_shuffles_against_golden(ab, golden):
    w8 = torch.from_numpy(golden["shufw_u8_in"].copy())
    assert np.array_equal(ab.shuffle_weight_f4(w8).numpy(), golden["f4_w_out"])
    s4 = torch.from_numpy(golden["f4_s_in"].copy())
    assert np.array_equal(ab.shuffle_scale_f4(s4, 7).numpy(), golden["f4_s_out_mx"])
    assert np.array_equal(ab.shuffle_scale_f4(s4, 8).numpy(), golden["f4_s_out_nv"])
    # and the packed order of the mxfp8 output scale is the inverse of the reference's unpacking
    packed = torch.from_numpy(golden["requant_fp8_scale_packed"].copy())
    assert np.array_equal(ab.unpack_mxfp8_out_scale(packed, 128, 256).view(torch.uint8).numpy(), golden["requant_fp8_scale"])


def test_table_lookup_rules(ab, tmp_path, monkeypatch):
    """The (gfx, cu_num, M, N, K) key: other targets' rows are ignored, padded-M buckets are tried after the
    exact M, merged files keep the fastest row, a legacy file without `gfx` falls back to a cu_num-only key,
    and edits take effect after a cache clear (reference: op_tests/test_gemm_codegen.py:292-390)."""
    from aiter_b200.config import TunedTable, get_cu_num, get_gfx

    gfx, cu = get_gfx(), get_cu_num()
    f1, f2 = tmp_path / "a.csv", tmp_path / "b.csv"
    _write_csv(f1, [f"{gfx},{cu},64,4096,4096,0,1,9.0,tc5_128x64_t_s4,0,0,0",
                    f"gfx950,256,1,4096,4096,0,3,1.0,amd_kernel,0,0,0",
                    f"{gfx},{cu},128,4096,4096,0,0,5.0,tc5_128x128_n_s4,0,0,0"])
    _write_csv(f2, [f"{gfx},{cu},64,4096,4096,0,2,3.0,tc5_128x64_t_s6,0,0,0"])
    monkeypatch.setenv("AITER_CONFIG_GEMM_A4W4", f"{f1}{os.pathsep}{f2}{os.pathsep}{tmp_path / 'missing.csv'}")
    table = TunedTable("a4w4")
    assert table.lookup(64, 4096, 4096)["kernelName"] == "tc5_128x64_t_s6"  # lowest `us` wins across files
    assert table.lookup(50, 4096, 4096)["kernelName"] == "tc5_128x64_t_s6"  # gl=0 bucket: 50 -> 64
    assert table.lookup(100, 4096, 4096)["kernelName"] == "tc5_128x128_n_s4"  # 100 -> 112 (miss) -> 128 (gl=1)
    assert table.lookup(1, 4096, 4096) is None  # the row tuned for another target (gfx950, 256 CUs) is ignored
    assert table.lookup(64, 4096, 1024) is None  # untuned shape: the caller falls back to the heuristic

    # edits take effect after a cache clear, without rebuilding anything
    _write_csv(f2, [f"{gfx},{cu},64,4096,4096,0,2,3.0,tc5_128x32_t_s8,0,0,0"])
    assert table.lookup(64, 4096, 4096)["kernelName"] == "tc5_128x64_t_s6"
    table.clear()
    assert table.lookup(64, 4096, 4096)["kernelName"] == "tc5_128x32_t_s8"

    # legacy schema without a gfx column: cu_num-only key
    legacy = tmp_path / "legacy.csv"
    _write_csv(legacy, [f"{cu},32,512,512,0,0,1.0,tc5_128x32_t_s4,0,0,0"],
               header="cu_num,M,N,K,kernelId,splitK,us,kernelName,tflops,bw,errRatio")
    monkeypatch.setenv("AITER_CONFIG_GEMM_A4W4", str(legacy))
    table.clear()
    assert table.lookup(32, 512, 512)["kernelName"] == "tc5_128x32_t_s4"


def test_a4w4_forwards_table_row_to_the_entry_point(ab, tmp_path, monkeypatch):
    """kernelName and splitK of the tuned row are forwarded verbatim; no row -> no kernel name and the
    library's own split choice (reference: op_tests/test_gemm_codegen.py:468-682)."""
    from aiter_b200 import gemm_op_a4w4
    from aiter_b200.config import get_cu_num, get_gfx

    csv = tmp_path / "a4w4.csv"
    _write_csv(csv, [f"{get_gfx()},{get_cu_num()},32,256,512,0,2,1.0,tc5_128x32_t_s4,0,0,0"])
    monkeypatch.setenv("AITER_CONFIG_GEMM_A4W4", str(csv))
    gemm_op_a4w4._table.clear()
    calls = []
    monkeypatch.setattr(gemm_op_a4w4._ffi, "call", lambda name, *args: calls.append((name, args)))
    A = torch.zeros((32, 256), dtype=torch.uint8)
    B = torch.zeros((256, 256), dtype=torch.uint8)
    S = torch.zeros((256, 16), dtype=torch.uint8)
    out = ab.gemm_a4w4(A, B, S, S)
    assert out.shape == (32, 256)
    name, args = calls[-1]
    assert name == "gemm_a4w4_asm" and args[5] == "tc5_128x32_t_s4" and args[10] == 2 and args[9] == 1
    assert args[4].shape == (32, 256)  # output rows padded to a multiple of 32
    ab.gemm_a4w4(torch.zeros((5, 256), dtype=torch.uint8), B, S, S)  # untuned M bucket
    name, args = calls[-1]
    assert args[5] is None and args[10] == -1 and args[4].shape == (32, 256)
    gemm_op_a4w4._table.clear()


def test_torch_library_ops_have_fake_implementations():
    """torch.ops.aiter.* trace on the meta device: output shape and dtype without touching a GPU."""
    import aiter_b200  # noqa: F401

    a = torch.empty(3, 5, 64, dtype=torch.uint8, device="meta")
    b = torch.empty(256, 64, dtype=torch.uint8, device="meta")
    s = torch.empty(256, 8, dtype=torch.uint8, device="meta")
    for op in (torch.ops.aiter.gemm_a4w4, torch.ops.aiter.gemm_a8w8_mxfp8, torch.ops.aiter.gemm_a8w4_mxfp8):
        o = op(a, b, s, s)
        assert o.shape == (3, 5, 256) and o.dtype == torch.bfloat16 and o.device.type == "meta"
    o = torch.ops.aiter.gemm_a16w16(torch.empty(7, 32, dtype=torch.bfloat16, device="meta"),
                                    torch.empty(48, 32, dtype=torch.bfloat16, device="meta"))
    assert o.shape == (7, 48)
    o = torch.ops.aiter.gemm_a8w8_blockscale(torch.empty(9, 256, dtype=torch.float8_e4m3fn, device="meta"),
                                             torch.empty(128, 256, dtype=torch.float8_e4m3fn, device="meta"),
                                             torch.empty(9, 2, device="meta"), torch.empty(1, 2, device="meta"))
    assert o.shape == (9, 128)
    o4 = torch.ops.aiter.gemm_a4w4o4(a, b, s, s)
    assert o4.shape == (3, 5, 128) and o4.dtype == torch.uint8
    o8, sc = torch.ops.aiter.gemm_a4w4o8(a, b, s, s, False, 0.5, 2.0)
    assert o8.shape == (3, 5, 256) and o8.dtype == torch.float8_e4m3fn and sc.shape == (3, 5, 2)
    o = torch.ops.aiter.gemm_nvfp4(a[0], b, s, s, 0.5, 2.0)
    assert o.shape == (5, 256) and o.dtype == torch.bfloat16
    o = torch.ops.aiter.batched_gemm_bf16(torch.empty(4, 7, 32, dtype=torch.bfloat16, device="meta"),
                                          torch.empty(4, 48, 32, dtype=torch.bfloat16, device="meta"))
    assert o.shape == (4, 7, 48) and o.dtype == torch.bfloat16


def test_fused_quantiser_wrappers_validate_arguments_on_cpu():
    """Argument rules of per_1x32_mx_quant_hip (aiter/ops/quant.py:486-597) that need no GPU."""
    import aiter_b200 as ab

    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="static per token"):
        ab.per_1x32_mx_quant_hip(x, scale=torch.zeros(1))
    with pytest.raises(ValueError, match="requires e8m0"):
        ab.per_1x32_mx_quant_hip(x, quant_dtype=ab.dtypes.fp4x2, scale_type=ab.dtypes.fp32)
    with pytest.raises(ValueError, match="unsupported quant_dtype"):
        ab.per_1x32_mx_quant_hip(x, quant_dtype=torch.int8)
    with pytest.raises(AssertionError):
        ab.per_1x32_mx_quant_hip(torch.zeros(4, 48, dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="fp4-only"):
        ab.per_1x32_f4_quant_hip(x, quant_dtype=ab.dtypes.fp8)
    assert ab.get_hip_quant(ab.QuantType.per_1x32) is ab.per_1x32_mx_quant_hip
    with pytest.raises(NotImplementedError):
        ab.get_hip_quant(ab.QuantType.per_Tensor)


def test_tuner_candidates_use_the_library_name_grammar():
    """Every candidate the tuner times has a name the library's documented grammar covers and a kernel id that
    follows `pair*1000 + swap*100 + bn_index*10 + stages` with the library's own tile-width menu."""
    import re

    import aiter_b200 as ab
    from aiter_b200 import tune

    menu_text = ab.kernel_list()
    widths = [int(m.group(2)) for m in re.finditer(r"id (\d+)\.\.: tile 128x(\d+) ", menu_text) if int(m.group(1)) < 100]
    assert widths == tune.BN_MENU
    grammar = re.compile(r"^tc5_(128|256)x(\d+)_[nt]_s\d(_k\d)?$")
    for fam, shapes in tune.BASELINE_SHAPES.items():
        for (M, N, K) in shapes:
            cands = tune.candidates(M, N, K, fam)
            assert cands, (fam, M, N, K)
            if fam.startswith("a8w8_blockscale"):  # these candidates are kernel names of the fp32-scale kernels
                assert all(c == "" or re.match(r"^bs_(fewrows|128x128|256x256|256x128)(_k\d)?$", c) for c in cands), cands
                continue
            for (pair, swap, bn, st, sk) in cands:
                assert bn in tune.BN_MENU and pair in (0, 1) and swap in (0, 1) and 0 <= st <= 8 and 0 <= sk <= 5
                assert not (pair and swap), "CTA-pair tiles are not built for the transposed (decode) orientation"
                assert grammar.match(tune.kernel_name(pair, swap, bn, st, sk)), tune.kernel_name(pair, swap, bn, st, sk)
                assert tune.kernel_id(pair, swap, bn, st) == pair * 1000 + swap * 100 + tune.BN_MENU.index(bn) * 10 + st


def test_tuner_worker_pool_survives_a_crash_and_a_hang(tmp_path, monkeypatch):
    """--mp: one worker process per GPU; a worker that exits with an error or outlives the watchdog loses only its
    unfinished shapes, which another worker gets once (reference: aiter/utility/mp_tuner.py:168-189).  Workers are
    replaced by a stand-in that needs no GPU."""
    import sys

    from aiter_b200 import tune

    marks = tmp_path / "marks"
    marks.mkdir()
    monkeypatch.setenv("AITER_B200_TUNE_WORKER_CMD", f"{sys.executable} {os.path.join(ROOT, 'tests', 'fake_tune_worker.py')}")
    monkeypatch.setenv("FAKE_WORKER_MARKS", str(marks))
    out = tmp_path / "tuned.csv"
    shapes = "1,256,512;13,256,512;2,256,512;17,256,512;3,256,512;19,256,512;4,256,512"
    rc = tune.main(["--family", "a4w4", "--shapes", shapes, "-o", str(out), "--mp", "3", "--timeout", "3"])
    assert rc == 1  # one shape has no valid result
    rows = tune.read_rows(str(out), "a4w4")
    got = sorted(k[2] for k in rows)
    assert got == [1, 2, 3, 4, 13, 17], got  # the crashed (13) and the hung (17) worker's shapes were retried; 19 failed twice
    assert all(r["kernelName"].startswith("tc5_128x64_n_s0_gpu") for r in rows.values())


def test_tuner_reads_shape_files_and_blockscale_names(tmp_path):
    from aiter_b200 import tune

    f = tmp_path / "untuned.csv"
    f.write_text("M,N,K,bias,dtype,outdtype,scaleAB,bpreshuffle\n64,1024,1024,False,torch.bfloat16,torch.bfloat16,False,False\n"
                 "64,1024,1024,False,torch.bfloat16,torch.bfloat16,False,False\n8,512,256,False,torch.bfloat16,torch.bfloat16,False,False\n")
    assert tune.shapes_from_file(str(f)) == [(64, 1024, 1024), (8, 512, 256)]
    names = tune.candidates(16, 4096, 4096, "a8w8_blockscale")
    assert "" in names and "bs_fewrows_k2" in names and "bs_128x128_k0" in names and "bs_256x256" not in names
    assert "bs_256x256" in tune.candidates(1024, 4096, 4096, "a8w8_blockscale_bpreshuffle")
    assert "bs_fewrows_k1" in tune.candidates(128, 4096, 4096, "a8w8_blockscale") and "bs_fewrows_k1" not in tune.candidates(300, 4096, 4096, "a8w8_blockscale")
    # beyond 256 rows the few-rows kernel is a candidate for narrow outputs only (up to 1024 rows by name)
    assert "bs_fewrows_k2" in tune.candidates(512, 512, 7168, "a8w8_blockscale") and "bs_256x128" in tune.candidates(512, 512, 7168, "a8w8_blockscale")
    assert "bs_fewrows_k0" not in tune.candidates(2048, 512, 7168, "a8w8_blockscale")


def test_blockscale_table_rows_do_not_leak_onto_e8m0_scaled_calls(ab):
    # the blockscale tables are tuned with fp32 scales; an e8m0-scaled call keeps only a few-rows row
    from aiter_b200 import gemm_op_a8w8 as g

    fp32_row = {"splitK": 1, "kernelName": "bs_128x128_k1"}
    few_row = {"splitK": 2, "kernelName": "bs_fewrows_k2"}
    assert g._blockscale_choice(fp32_row, False, 128, 4096, 4096) == (1, "bs_128x128_k1")
    assert g._blockscale_choice(few_row, True, 16, 4096, 4096) == (2, "bs_fewrows_k2")
    split, name = g._blockscale_choice(fp32_row, True, 128, 4096, 4096)
    assert split == 0 and not name.startswith("bs_")
    assert g._blockscale_choice({"splitK": 0, "kernelName": "bs_256x256"}, True, 16, 4096, 4096) == (0, "")
    assert g._blockscale_choice(None, False, 5, 6, 7) == (0, "")
    # 65..256 rows whose tiles of 64 rows fit the machine at once: no name, the launcher keeps the call on the few-rows
    # kernel (one launch); beyond that the MXFP8 table's row for the shape is passed on
    assert g._blockscale_choice({"splitK": 0, "kernelName": ""}, True, 128, 4096, 4096) == (0, "")
    assert g._blockscale_choice(fp32_row, True, 256, 4096, 4096) == (0, "")
    split, name = g._blockscale_choice(None, True, 1024, 4096, 4096)
    assert split == 0 and name.startswith("tc5_")
    split, name = g._blockscale_choice(None, True, 256, 16384, 4096)  # 128 x 4 tiles: more than the machine has SMs
    assert split == 0 and not name.startswith("bs_")
