"""Generate golden vectors from the reference's own Python functions.

Run once where the reference sources are mounted:

    python tests/golden/gen_golden.py /path/to/reference

The reference package cannot be imported as a whole without its GPU stack, so the
numerics modules (aiter/utility/{aiter_types,dtypes,mx_types,fp4_utils}.py and
aiter/ops/shuffle.py) are loaded file by file behind a handful of stub modules - the
same trick the reference's host-only tests use
(op_tests/tuning_tests/test_asm_splitk_guard.py:20-80).  The two thin compositions in
aiter/ops/quant.py (per_1x32_f4_quant :157-204, per_1x32_f8_scale_f8_quant :272-315)
cannot be imported (the file pulls in Triton kernels at import), so they are composed
here from the imported primitives exactly as those lines do.

Outputs (committed): tests/golden/mx_golden.npz - small, a few hundred KB.
"""
from __future__ import annotations

import importlib.util
import logging
import os
import sys
import types

import numpy as np
import torch


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    m.__path__ = []  # behave like a package
    sys.modules[name] = m
    return m


def load_reference(ref_root: str):
    def compile_ops(*_a, **_k):
        def deco(fn):
            return fn

        return deco

    _stub("aiter", logger=logging.getLogger("aiter"))
    _stub("aiter.jit")
    _stub("aiter.jit.core", compile_ops=compile_ops, get_module=lambda *_: None)
    _stub("aiter.jit.utils")
    _stub(
        "aiter.jit.utils.chip_info",
        get_gfx=lambda: "gfx950",
        get_gfx_runtime=lambda: "gfx950",
        get_cu_num=lambda: 256,
    )
    _stub("aiter.jit.utils.torch_guard", torch_compile_guard=lambda **_k: (lambda f: f))
    _stub("aiter.ops")
    _stub("aiter.ops.enum", ActivationType=object, QuantType=object)
    _stub("aiter.utility")

    def load(modname, rel):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    load("aiter.utility.aiter_types", "aiter/utility/aiter_types.py")
    dtypes = load("aiter.utility.dtypes", "aiter/utility/dtypes.py")
    sys.modules["aiter.utility"].dtypes = dtypes
    load("aiter.utility.mx_types", "aiter/utility/mx_types.py")
    fp4_utils = load("aiter.utility.fp4_utils", "aiter/utility/fp4_utils.py")
    shuffle = load("aiter.ops.shuffle", "aiter/ops/shuffle.py")
    return dtypes, fp4_utils, shuffle


def ref_per_1x32_f4_quant(fp4_utils, x):
    """aiter/ops/quant.py:180-204 with round_mode = RoundUp, shuffle=False."""
    from aiter.utility.mx_types import MX_DEFAULT_ROUND_MODE, MxDtypeInt

    shape = x.shape
    xb = x.view(-1, 32)
    max_abs = torch.amax(torch.abs(xb.float()), 1)
    sb = fp4_utils.f32_to_mx_e8m0_scale(max_abs, mode=MX_DEFAULT_ROUND_MODE, dtype=MxDtypeInt.FP4_E2M1)
    sf = fp4_utils.e8m0_to_f32(sb)
    y = fp4_utils.f32_to_mxfp4(xb.float() / sf.view(-1, 1))
    return y.view(torch.uint8).view(shape[0], -1), sb.view(torch.uint8).view(shape[0], -1)


def ref_per_1x32_f8_quant(fp4_utils, x):
    """aiter/ops/quant.py:282-315 with scale_type = e8m0, shuffle=False."""
    from aiter.utility.mx_types import MX_DEFAULT_ROUND_MODE, MxDtypeInt

    shape = x.shape
    xb = x.view(-1, 32)
    max_abs = torch.amax(torch.abs(xb.float()), 1)
    sb = fp4_utils.f32_to_mx_e8m0_scale(max_abs, mode=MX_DEFAULT_ROUND_MODE, dtype=MxDtypeInt.FP8_E4M3)
    sf = fp4_utils.e8m0_to_f32(sb)
    y = (xb.float() / sf.view(-1, 1)).view(shape).to(torch.float8_e4m3fn)
    return y.view(torch.uint8), sb.view(torch.uint8).view(shape[0], -1)


def ref_gemm_a4w4(fp4_utils, x, w, xs, ws):
    """op_tests/test_gemm_a4w4.py:23-39."""
    m, n = x.shape[0], w.shape[0]
    xf = fp4_utils.mxfp4_to_f32(x) * fp4_utils.e8m0_to_f32(xs[:m].repeat_interleave(32, dim=1))
    wf = fp4_utils.mxfp4_to_f32(w) * fp4_utils.e8m0_to_f32(ws[:n].repeat_interleave(32, dim=1))
    return torch.mm(xf, wf.T).to(torch.bfloat16)


def ref_gemm_nvfp4(fp4_utils, xq, wq, xs, ws, gA, gB, noscale=False):
    """op_tests/test_f4gemm.py:122-133 (run_torch_nvfp4): fp32 result, e4m3 scales per 16 elements, per-tensor factors."""
    x_f32 = fp4_utils.mxfp4_to_f32(xq)
    w_f32 = fp4_utils.mxfp4_to_f32(wq)
    if noscale:
        return float(gA) * float(gB) * (x_f32 @ w_f32.T)
    xsf = xs.view(torch.float8_e4m3fn).to(torch.float32).repeat_interleave(16, dim=1)
    wsf = ws.view(torch.float8_e4m3fn).to(torch.float32).repeat_interleave(16, dim=1)
    return float(gA) * float(gB) * (x_f32 * xsf) @ (w_f32 * wsf).T


def ref_gemm_mxfp8(fp4_utils, intype, a, b, sa, sb):
    """op_tests/test_mxfp8fp4gemm.py:63-72."""
    af = a.view(torch.float8_e4m3fn).to(torch.float32)
    bf = fp4_utils.mxfp4_to_f32(b) if intype == "a8w4" else b.view(torch.float8_e4m3fn).to(torch.float32)
    saf = fp4_utils.e8m0_to_f32(sa).repeat_interleave(32, dim=1)
    sbf = fp4_utils.e8m0_to_f32(sb).repeat_interleave(32, dim=1)
    return ((af * saf) @ (bf * sbf).T).to(torch.bfloat16)


def ref_gemm_blockscale(fp4_utils, x, weight, x_scale, w_scale, block_shape=(128, 128)):
    """op_tests/test_gemm_a8w8_blockscale.py:30-56 (einops.rearrange written out as permute + reshape)."""
    block_n, block_k = block_shape
    m, k = x.shape
    n = weight.shape[0]
    scale_n, scale_k = (n + block_n - 1) // block_n, (k + block_k - 1) // block_k
    if x_scale.dtype == torch.float8_e8m0fnu:
        x_scale = fp4_utils.e8m0_to_f32(x_scale)
    if w_scale.dtype == torch.float8_e8m0fnu:
        w_scale = fp4_utils.e8m0_to_f32(w_scale)
    xf = (x.to(x_scale.dtype).view(m, k // block_k, block_k) * x_scale.unsqueeze(-1)).view(m, k)
    ws = w_scale.view(-1, 1).repeat(1, block_n * block_k).view(scale_n, scale_k, block_n, block_k)
    ws = ws.permute(0, 2, 1, 3).reshape(scale_n * block_n, scale_k * block_k)[:n, :k]
    wf = weight.to(ws.dtype) * ws
    return torch.nn.functional.linear(xf.to(torch.float32), wf.to(torch.float32)).to(torch.bfloat16)


def ref_quant_mxfp8_blockN(fp4_utils, MxDtypeInt, x_f32, block=128):
    """op_tests/test_f4gemm.py:73-88: fp8 e4m3 data + one RoundUp E8M0 scale per 128 output columns."""
    M, N = x_f32.shape
    xb = x_f32.reshape(M, N // block, block)
    amax = xb.abs().amax(dim=-1).clamp(min=torch.finfo(torch.float32).tiny)
    scale = fp4_utils.f32_to_mx_e8m0_scale(amax, mode=1, dtype=MxDtypeInt.FP8_E4M3)
    q = (xb / fp4_utils.e8m0_to_f32(scale).unsqueeze(-1)).reshape(M, N).to(torch.float8_e4m3fn)
    return q, scale


def ref_pack_mxfp8_out_scale(rm):
    """Inverse of unpack_mxfp8_out_scale (aiter/ops/gemm_op_a4w4.py:365-380): row-major [M, N/128] -> the packed
    (M/64, N/128, 16, 4) byte order."""
    M, sn = rm.shape
    return rm.view(torch.uint8).reshape(M // 64, 4, 16, sn).permute(0, 3, 2, 1).contiguous().reshape(M, sn)


def bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main(ref_root: str, out_path: str):
    dtypes, fp4_utils, shuffle = load_reference(ref_root)
    g = {}

    # ---- scalar known answers: e2m1 rounding, e8m0 scale boundaries, e4m3 cast
    probe = torch.tensor(
        [0.0, -0.0, 0.1, -0.1, 0.25, -0.25, 0.2500001, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5,
         3.0, 3.5, 4.0, 5.0, 5.9999, 6.0, 7.0, -7.0, 1e4, 1e-10, -3.0, 0.7499999, 2.4999998, 4.9999995],
        dtype=torch.float32,
    )
    g["e2m1_probe_in"] = probe.numpy()
    g["e2m1_probe_out"] = fp4_utils._f32_to_floatx_unpacked(probe, 2, 1).numpy()
    g["e2m1_lut"] = fp4_utils.mxfp4_to_f32(torch.arange(256, dtype=torch.uint8).view(-1, 1)).numpy()

    from aiter.utility.mx_types import MX_DEFAULT_ROUND_MODE, MxDtypeInt

    torch.manual_seed(1)
    amax = torch.cat(
        [
            torch.tensor([0.0, 6.0, 12.0, 6.0000005, 5.9999995, 448.0, 896.0, 448.00003, 1e-38, 1e-45, 3e38, 1.0, 3.0, 0.75]),
            6.0 * torch.exp2(torch.arange(-20, 20).float()),
            448.0 * torch.exp2(torch.arange(-20, 20).float()),
            torch.rand(2000) * 100,
            torch.exp2(torch.rand(2000) * 60 - 30),
        ]
    ).float()
    g["amax_in"] = amax.numpy()
    g["amax_e8m0_fp4"] = fp4_utils.f32_to_mx_e8m0_scale(amax, mode=MX_DEFAULT_ROUND_MODE, dtype=MxDtypeInt.FP4_E2M1).view(torch.uint8).numpy()
    g["amax_e8m0_fp8"] = fp4_utils.f32_to_mx_e8m0_scale(amax, mode=MX_DEFAULT_ROUND_MODE, dtype=MxDtypeInt.FP8_E4M3).view(torch.uint8).numpy()
    allb = torch.arange(256, dtype=torch.uint8)
    g["e8m0_to_f32_bits"] = fp4_utils.e8m0_to_f32(allb).view(torch.int32).numpy().view(np.uint32)

    e4 = torch.cat(
        [
            torch.tensor([0.0, -0.0, 2.0**-9, 2.0**-10, 1.5 * 2.0**-10, 3 * 2.0**-10, 448.0, 449.0, 463.9, 464.0, 479.9, -448.0, 0.0175, 17.5]),
            torch.randn(4000) * 100,
            torch.exp2(torch.rand(2000) * 20 - 12),
        ]
    ).float()
    g["e4m3_in"] = e4.numpy()
    g["e4m3_out"] = e4.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    g["e4m3_decode_bits"] = allb.view(torch.float8_e4m3fn).to(torch.float32).view(torch.int32).numpy().view(np.uint32)

    # ---- block quantisers on seeded bf16 data (+ edge rows)
    torch.manual_seed(0)
    x = torch.randn(48, 256, dtype=torch.float32).to(torch.bfloat16)
    x[0, :32] = 0  # all-zero block
    x[1, :32] = 1e4
    x[2, :32] = 1e-10
    x[3, :32] = -3.0
    x[4, :64] = torch.linspace(-8, 8, 64).to(torch.bfloat16)
    g["quant_in_bf16"] = bits16(x)
    q4, s4 = ref_per_1x32_f4_quant(fp4_utils, x)
    g["quant_fp4_data"], g["quant_fp4_scale"] = q4.numpy(), s4.numpy()
    q8, s8 = ref_per_1x32_f8_quant(fp4_utils, x)
    g["quant_fp8_data"], g["quant_fp8_scale"] = q8.numpy(), s8.numpy()

    # ---- shuffles on index-coded tensors
    w8 = (torch.arange(64 * 128) % 251).to(torch.uint8).view(64, 128)
    g["shufw_u8_in"] = w8.numpy()
    g["shufw_u8_out"] = shuffle.shuffle_weight(w8, layout=(16, 16)).numpy()
    w16 = torch.arange(32 * 64, dtype=torch.int16).view(32, 64)
    g["shufw_i16_in"] = w16.numpy()
    g["shufw_i16_out"] = shuffle.shuffle_weight(w16, layout=(16, 16)).numpy()
    sc = (torch.arange(512 * 16) % 253).to(torch.uint8).view(512, 16)
    g["shufs_in"] = sc.numpy()
    g["shufs_out"] = shuffle.shuffle_scale(sc).numpy()  # exact multiples: no uninitialised padding
    sc2 = (torch.arange(40 * 12) % 253).to(torch.uint8).view(40, 12)
    g["shufs_ragged_in"] = sc2.numpy()
    g["shufs_ragged_out"] = shuffle.shuffle_scale(sc2).numpy()  # padding is uninitialised: compare valid slots only
    a8 = (torch.arange(6 * 256) % 251).to(torch.uint8).view(6, 256)
    g["g1250_a_in"], g["g1250_a_out"] = a8.numpy(), shuffle.shuffle_mxfp8fp4_a(a8).numpy()
    g["g1250_b_in"], g["g1250_b_out"] = w8.numpy(), shuffle.shuffle_mxfp8fp4_b(w8).numpy()
    s3 = (torch.arange(40 * 8) % 253).to(torch.uint8).view(40, 8)
    g["g1250_s_in"], g["g1250_s_out"] = s3.numpy(), shuffle.shuffle_mxfp8fp4_scale(s3).numpy()

    g["f4_w_out"] = shuffle.shuffle_weight_f4(w8).numpy()
    s4 = (torch.arange(64 * 16) % 253).to(torch.uint8).view(64, 16)
    g["f4_s_in"] = s4.numpy()
    g["f4_s_out_mx"], g["f4_s_out_nv"] = shuffle.shuffle_scale_f4(s4, 7).numpy(), shuffle.shuffle_scale_f4(s4, 8).numpy()

    # ---- GEMM references on small seeded problems
    torch.manual_seed(0)
    a = (torch.randn(64, 1024) * 0.1).to(torch.bfloat16)
    b = (torch.randn(96, 1024) * 0.1).to(torch.bfloat16)
    g["gemm_bf16_a"], g["gemm_bf16_b"] = bits16(a), bits16(b)
    g["gemm_bf16_out"] = bits16(torch.nn.functional.linear(a.float(), b.float()).to(torch.bfloat16))

    xa = torch.randn(33, 512).to(torch.bfloat16)
    wb = torch.randn(80, 512).to(torch.bfloat16)
    xa4, xs4 = ref_per_1x32_f4_quant(fp4_utils, xa)
    wb4, ws4 = ref_per_1x32_f4_quant(fp4_utils, wb)
    g["gemm_a4w4_x"], g["gemm_a4w4_w"], g["gemm_a4w4_xs"], g["gemm_a4w4_ws"] = xa4.numpy(), wb4.numpy(), xs4.numpy(), ws4.numpy()
    g["gemm_a4w4_out"] = bits16(ref_gemm_a4w4(fp4_utils, xa4, wb4, xs4, ws4))
    xa8, xs8 = ref_per_1x32_f8_quant(fp4_utils, xa)
    wb8, ws8 = ref_per_1x32_f8_quant(fp4_utils, wb)
    g["gemm_a8w8_x"], g["gemm_a8w8_w"], g["gemm_a8w8_xs"], g["gemm_a8w8_ws"] = xa8.numpy(), wb8.numpy(), xs8.numpy(), ws8.numpy()
    g["gemm_a8w8_out"] = bits16(ref_gemm_mxfp8(fp4_utils, "a8w8", xa8, wb8, xs8, ws8))
    g["gemm_a8w4_out"] = bits16(ref_gemm_mxfp8(fp4_utils, "a8w4", xa8, wb4, xs8, ws4))

    # ---- fp8 x fp8 with 128-block scales (fp32 and e8m0 scale tensors)
    torch.manual_seed(1)
    bx = (torch.randn(40, 384) * 2).to(torch.float8_e4m3fn)
    bw = (torch.randn(200, 384) * 2).to(torch.float8_e4m3fn)
    bxs = torch.rand(40, 3) + 0.25
    bws = torch.rand(2, 3) + 0.25
    g["bs_x"], g["bs_w"] = bx.view(torch.uint8).numpy(), bw.view(torch.uint8).numpy()
    g["bs_xs"], g["bs_ws"] = bxs.numpy(), bws.numpy()
    g["bs_out"] = bits16(ref_gemm_blockscale(fp4_utils, bx, bw, bxs, bws))
    exs = torch.randint(124, 131, (40, 3), dtype=torch.uint8)
    ews = torch.randint(124, 131, (2, 3), dtype=torch.uint8)
    g["bs_xs_e8m0"], g["bs_ws_e8m0"] = exs.numpy(), ews.numpy()
    g["bs_out_e8m0"] = bits16(ref_gemm_blockscale(fp4_utils, bx, bw, exs.view(torch.float8_e8m0fnu), ews.view(torch.float8_e8m0fnu)))

    # ---- low-precision GEMM outputs: the re-quantisation of an fp32 result (op_tests/test_f4gemm.py:73-88,211-217)
    torch.manual_seed(2)
    y = torch.randn(128, 256) * torch.exp2(torch.randint(-6, 7, (128, 1)).float())
    y[0, :128] = 0.0        # an all-zero 128-column block
    y[1, :128] = 448.0      # exact maximum: the scale must not bump
    y[2, 5] = 3.0e4
    g["requant_in"] = y.numpy()
    q8, s8 = ref_quant_mxfp8_blockN(fp4_utils, MxDtypeInt, y)
    g["requant_fp8_data"], g["requant_fp8_scale"] = q8.view(torch.uint8).numpy(), s8.view(torch.uint8).numpy()
    g["requant_fp8_scale_packed"] = ref_pack_mxfp8_out_scale(s8).numpy()
    g["requant_fp4_data"] = fp4_utils.f32_to_mxfp4(y).view(torch.uint8).numpy()

    # ---- NVFP4 inputs: packed e2m1 data, e4m3 scales per 16 elements (positive, around 0.34 as the reference's bench
    # initialiser draws them, op_tests/test_f4gemm.py:175-181), per-tensor factors
    torch.manual_seed(3)
    nx = torch.randint(0, 256, (48, 256), dtype=torch.uint8)   # [48, K=512] packed
    nw = torch.randint(0, 256, (64, 256), dtype=torch.uint8)
    nxs = (torch.randn(48, 32) * 0.08 + 0.34375).clamp(0.015625, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    nws = (torch.randn(64, 32) * 0.08 + 0.34375).clamp(0.015625, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    g["nv_x"], g["nv_w"], g["nv_xs"], g["nv_ws"] = nx.numpy(), nw.numpy(), nxs.numpy(), nws.numpy()
    g["nv_g"] = np.array([0.75, 1.3], dtype=np.float64)
    g["nv_out_f32"] = ref_gemm_nvfp4(fp4_utils, nx, nw, nxs, nws, 0.75, 1.3).numpy()
    g["nv_out_bf16"] = bits16(ref_gemm_nvfp4(fp4_utils, nx, nw, nxs, nws, 0.75, 1.3).to(torch.bfloat16))
    g["nv_out_noscale_f32"] = ref_gemm_nvfp4(fp4_utils, nx, nw, nxs, nws, 0.75, 1.3, noscale=True).numpy()

    np.savez_compressed(out_path, **g)
    print("wrote", out_path, os.path.getsize(out_path), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/gen_golden.py /path/to/reference [output.npz]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "mx_golden.npz"))
