"""Batched bf16 GEMM (batched_gemm_bf16 / _CK / _tune): every entry of the batch against the numpy oracle, in both
storage orders the reference's test uses ([b, m, k] contiguous and the transposed view of [m, b, k]), as one launch."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as ox
from tests.helpers import bf16_bits, check

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import aiter_b200

    return aiter_b200


def _ints(shape, seed):
    # the reference's test draws integers in [-20, 20) (op_tests/test_batched_gemm_bf16.py:41-55)
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-20, 20, shape, generator=g).to(torch.bfloat16)


def _ref(x, w, i):
    return ox.gemm_a16w16_ref(bf16_bits(x[i].contiguous()), bf16_bits(w[i].contiguous()))


@pytest.mark.parametrize("b,m,n,k", [(16, 1, 1280, 8192), (4, 40, 320, 512), (3, 300, 200, 264), (2, 1024, 768, 1024), (1, 64, 256, 128)])
@pytest.mark.parametrize("layout", ["bmn", "mbn"])
def test_batched_gemm_bf16(ab, b, m, n, k, layout):
    w = _ints((b, n, k), 1)
    if layout == "mbn":
        x = _ints((m, b, k), 2).transpose(0, 1)  # logically [b, m, k], stored [m, b, k]
        y = torch.full((m, b, n), float("nan"), dtype=torch.bfloat16, device="cuda").transpose(0, 1)
    else:
        x = _ints((b, m, k), 2)
        y = torch.full((b, m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    xd = x.cuda() if layout == "bmn" else x.transpose(0, 1).contiguous().cuda().transpose(0, 1)
    before = ab.launch_count()
    out = ab.batched_gemm_bf16(xd, w.cuda(), y)
    assert ab.launch_count() == before + 1, "the batch must be one launch"
    assert out.data_ptr() == y.data_ptr() and out.shape == (b, m, n)
    for i in range(b):
        check(_ref(x, w, i), out[i], what=f"batched bf16 {layout} entry {i} of {b}x{m}x{n}x{k}")
    assert ab.device_status(0) == (0, 0, 0, 0)


def test_batched_gemm_bf16_ck_form_bias_and_tune(ab):
    b, m, n, k = 4, 96, 384, 1024
    x, w = _ints((b, m, k), 3), _ints((b, n, k), 4)
    out = ab.batched_gemm_bf16_CK(x.cuda(), w.cuda())
    assert out.shape == (b, m, n) and out.dtype == torch.bfloat16
    for i in range(b):
        check(_ref(x, w, i), out[i], what=f"batched_gemm_bf16_CK entry {i}")
    # fp16 output; a bias must have the output's dtype and, as in the reference's CK instances, is not added
    xs, ws = (x * 0.05).to(torch.bfloat16), (w * 0.05).to(torch.bfloat16)
    bias = torch.ones(n, dtype=torch.float16, device="cuda")
    o16 = ab.batched_gemm_bf16_CK(xs.cuda(), ws.cuda(), bias=bias, dtype=torch.float16)
    assert o16.dtype == torch.float16
    for i in range(b):
        ref = ox.gemm_f32(ox.bf16_bits_to_f32(bf16_bits(xs[i])), ox.bf16_bits_to_f32(bf16_bits(ws[i])))
        got = o16[i].float().cpu().numpy()
        assert np.all(np.abs(got - ref) <= 1e-2 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()
    with pytest.raises(RuntimeError, match="same dtype"):
        ab.batched_gemm_bf16(x.cuda(), w.cuda(), torch.empty(b, m, n, dtype=torch.bfloat16, device="cuda"), bias=bias)
    # the _tune form: a tile id of the menu and log2 of the K split (tickets and partial tiles are per (entry, tile))
    for kid, split in ((20, 0), (20, 2), (124, 1), (1040, 0)):
        y = torch.full((b, m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        ab.batched_gemm_bf16_tune(x.cuda(), w.cuda(), y, kid, split)
        for i in range(b):
            check(_ref(x, w, i), y[i], what=f"batched_gemm_bf16_tune id {kid} split {split} entry {i}")
    with pytest.raises(RuntimeError, match="not found"):
        ab.batched_gemm_bf16_tune(x.cuda(), w.cuda(), y, 99999, 0)
    with pytest.raises(RuntimeError, match="batch mismatch"):
        ab.batched_gemm_bf16(x.cuda(), w[:2].cuda(), y)
    assert ab.device_status(0) == (0, 0, 0, 0)
