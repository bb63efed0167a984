"""The tuner end to end on the GPU: one small shape per family is tuned into a temporary table, the table is loaded
back through its AITER_CONFIG_GEMM_* variable, and the public operator - now dispatched by that row - is checked
against a reference.  Also --compare / --update_improved and --run_config."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = {
    "a4w4": (48, 512, 1024),
    "a8w8_mxfp8": (16, 512, 1024),
    "a8w4_mxfp8": (160, 512, 1024),
    "bf16": (64, 512, 512),
    "a8w8_blockscale": (24, 512, 1024),
    "a8w8_blockscale_bpreshuffle": (200, 512, 1024),
}


@pytest.mark.parametrize("family", sorted(SHAPES))
def test_tune_then_dispatch_through_the_table(family, tmp_path, monkeypatch):
    from aiter_b200 import config, tune

    M, N, K = SHAPES[family]
    out = tmp_path / f"{family}.csv"
    assert tune.main(["--family", family, "--shapes", f"{M},{N},{K}", "-o", str(out)]) == 0
    rows = tune.read_rows(str(out), family)
    assert len(rows) == 1
    row = next(iter(rows.values()))
    assert float(row["us"]) > 0 and float(row.get("errRatio", row.get("err_ratio", 0)) or 0) == 0.0
    # the production operator, steered by that file
    dev = torch.device("cuda", 0)
    try:
        res = tune.run_config(family, [(M, N, K)], dev, str(out), verbose=False)
        assert res[(M, N, K)] is not None, "the tuned row did not run or missed the tolerance"
        found = tune._family_tables(family)[0].lookup(M, N, K, *((False, "torch.bfloat16", "torch.bfloat16", False, False) if family == "bf16" else ()))
        assert found is not None and str(found["kernelName"] or "") == str(row["kernelName"] or "")
    finally:
        tune.use_table(family, None)
    assert os.environ.get(config.TABLES[tune.FAMILIES[family][0]][0]) is None


def test_compare_and_update_improved(tmp_path, capsys):
    from aiter_b200 import tune

    out = tmp_path / "a8w8.csv"
    # a deliberately poor row first: a 16-wide tile with a 4-stage pipeline and no K split for a 4096-deep problem
    out.write_text("gfx,cu_num,M,N,K,kernelId,splitK,us,kernelName,tflops,bw,errRatio\n"
                   "sm_100a,148,16,512,4096,14,0,99.0,tc5_128x16_n_s4_k0,0.1,1.0,0.0\n")
    try:
        assert tune.main(["--family", "a8w8_mxfp8", "--shapes", "16,512,4096", "-o", str(out), "--compare", "--update_improved",
                          "--min_improvement_pct", "1"]) == 0
    finally:
        tune.use_table("a8w8_mxfp8", None)
    text = capsys.readouterr().out
    assert "before" in text and "after" in text
    rows = tune.read_rows(str(out), "a8w8_mxfp8")
    assert os.path.exists(str(out) + ".compare_candidate.csv")
    row = next(iter(rows.values()))
    if "improved" in text:
        assert row["kernelName"] != "tc5_128x16_n_s4_k0"
    # --run_config on the resulting table: shapes and kernels come from the file
    try:
        assert tune.main(["--family", "a8w8_mxfp8", "--run_config", str(out)]) == 0
    finally:
        tune.use_table("a8w8_mxfp8", None)
