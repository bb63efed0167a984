"""bf16 front door: gemm_a16w16 / tgemm.mm (reference: aiter/tuned_gemm.py:207-300,354-418,672-730).

The bf16 table row for (M, N, K, bias, dtype, outdtype, scaleAB, bpreshuffle) names a `libtype`; the
back-ends kept here are the ones that exist on this hardware: "opus" and "asm" (both served by the
tcgen05 kernel family, by kernel id resp. kernel name).  A row that names any other back-end (the
reference's tables also know "torch", "hipblaslt", "triton", ...) is an error: nothing here dispatches to
another library.  An untuned shape runs the library's own heuristic.
"""
from __future__ import annotations

import logging
import os

import torch
from torch import Tensor

from . import dtypes
from .config import get_cu_num, get_gfx  # noqa: F401
from .gemm_op_a16w16 import _bf16_table, gemm_a16w16_asm, opus_gemm, opus_gemm_a16w16_tune

logger = logging.getLogger("aiter")


def get_GEMM_A16W16_config(M: int, N: int, K: int, bias: bool, dtype: str, otype: str, scaleAB: bool = False,
                           bpreshuffle: bool = False):
    cfg = _bf16_table.lookup(M, N, K, bias, str(dtype), str(otype), scaleAB, bpreshuffle)
    if cfg is not None:
        return cfg
    default = {"libtype": "asm" if bpreshuffle else "opus", "solidx": -1, "splitK": None, "kernelName": None}
    if bpreshuffle:
        default["bpreshuffle"] = True
    logger.info(f"shape is M:{M}, N:{N}, K:{K} {dtype=} {otype=} {bias=}, {scaleAB=}, {bpreshuffle=}, not found tuned config, "
                f"will use default config! using {default['libtype']} heuristic")
    return default


def asm_gemm(inp, weights, solidx, bias=None, otype=None, scale_a=None, scale_b=None, scale_c=None, bpreshuffle=False, config=None):
    kernelName = config.get("kernelName") if config else None
    splitK = config.get("splitK") if config else None
    out = torch.empty(inp.shape[0], weights.shape[0], dtype=otype, device=inp.device)
    return gemm_a16w16_asm(inp, weights, out, bias, splitK, kernelName, bpreshuffle)


def opus_gemm_backend(inp, weights, solidx, bias=None, otype=None, scale_a=None, scale_b=None, scale_c=None, bpreshuffle=False, config=None):
    assert scale_a is None and scale_b is None and scale_c is None, "opus_gemm does not support scaling"
    assert not bpreshuffle, "opus_gemm does not support bpreshuffle"
    m, n = inp.shape[0], weights.shape[0]
    Y = torch.empty(m, n, dtype=otype or inp.dtype, device=inp.device)
    if solidx is None or int(solidx) < 0:
        opus_gemm(inp.unsqueeze(0), weights.unsqueeze(0), Y.unsqueeze(0), None, None, None, bias)
    else:
        splitK = int(config.get("splitK") or 0) if config is not None else 0
        opus_gemm_a16w16_tune(inp.unsqueeze(0), weights.unsqueeze(0), Y.unsqueeze(0), bias=bias, kernelId=int(solidx), splitK=splitK)
    return Y


solMap = {"asm": asm_gemm, "opus": opus_gemm_backend}


def gemm_a16w16(A: Tensor, B: Tensor, bias: Tensor | None = None, otype: torch.dtype | None = None,
                scale_a: Tensor | None = None, scale_b: Tensor | None = None, scale_c: Tensor | None = None) -> Tensor:
    """out[.., N] = A[.., K] @ B[N, K]^T (+ bias).  A weight produced by shuffle_weight (tagged `.is_shuffled`)
    is consumed in its shuffled form."""
    if scale_a is not None or scale_b is not None or scale_c is not None:
        raise NotImplementedError("per-tensor scaled inputs are outside this library's GEMM path")
    bpreshuffle = bool(getattr(B, "is_shuffled", False))
    if A.dim() >= 3:
        inp_view, batched = A.reshape(-1, A.size(-1)), True
    else:
        inp_view, batched = A, False
    m, k = inp_view.shape
    n = B.shape[0]
    otype = otype if otype is not None else inp_view.dtype
    config = get_GEMM_A16W16_config(m, n, k, bias is not None, str(inp_view.dtype), str(otype), False, bpreshuffle)
    libtype = config["libtype"]
    if libtype not in solMap:
        raise RuntimeError(f"bf16 table row for ({m},{n},{k}) names back-end '{libtype}', which does not exist in this build")
    # the kernels write bf16 or fp32 themselves (fp32 straight from the accumulator); other output types are a cast of bf16
    kernel_otype = otype if otype in (dtypes.bf16, torch.float32) else dtypes.bf16
    out = solMap[libtype](inp_view, B, config.get("solidx"), bias, kernel_otype, None, None, None, bpreshuffle, config=config)
    if batched:
        out = out.view(*A.shape[:-1], n)
    if out.dtype != otype:
        out = out.to(otype)
    if tgemm.save_gemm == 1:
        tgemm.record_shape(m, n, k, bias is not None, inp_view.dtype, otype, False, bpreshuffle)
    return out


class TunedGemm:
    """`tgemm.mm(inp, weights, bias=None, otype=None)` - the call serving frameworks make."""

    def __init__(self):
        self.save_gemm = int(os.environ.get("AITER_TUNE_GEMM", "0"))
        self.untune_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs", "bf16_untuned_gemm.csv")
        self.seen = set()

    def record_shape(self, *key):
        """AITER_TUNE_GEMM=1: append shapes that reach the front door to the untuned list for the tuner."""
        if key in self.seen:
            return
        self.seen.add(key)
        new = not os.path.exists(self.untune_path)
        with open(self.untune_path, "a") as f:
            if new:
                f.write("M,N,K,bias,dtype,outdtype,scaleAB,bpreshuffle\n")
            f.write(",".join(str(v) for v in key) + "\n")

    def mm(self, inp: Tensor, weights: Tensor, bias: Tensor | None = None, otype: torch.dtype | None = None,
           scale_a: Tensor | None = None, scale_b: Tensor | None = None, scale_c: Tensor | None = None):
        return gemm_a16w16(inp, weights, bias=bias, otype=otype, scale_a=scale_a, scale_b=scale_b, scale_c=scale_c)


tgemm = TunedGemm()
