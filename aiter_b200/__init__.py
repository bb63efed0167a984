"""aiter_b200 - the quantised-GEMM hot path of the aiter operator library, rebuilt for B200 (sm_100a).

Same operator names and argument meaning as the reference package; underneath, hand-written
tcgen05 / TMA kernels behind a C ABI (include/aiter_b200.h).  Importing this package loads the
CUDA library and fails loudly when it has not been built.
"""
import logging
import os

logger = logging.getLogger("aiter")
if not logger.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[aiter] %(levelname)s: %(message)s"))
    logger.addHandler(_h)
    logger.setLevel(getattr(logging, os.getenv("AITER_LOG_LEVEL", "WARNING").upper(), logging.WARNING))
    logger.propagate = False

from . import dtypes, fp4_utils  # noqa: E402
from ._ffi import debug_wait_control, device_status, get_padded_m, heuristic_name, kernel_list, launch_count, noalloc_status  # noqa: E402,F401
from .dtypes import MX_DEFAULT_ROUND_MODE, MxDtype, MxScaleRoundMode, QuantType  # noqa: E402,F401
from .gemm_op_a4w4 import (  # noqa: E402,F401
    gemm_a4w4,
    gemm_a4w4_asm,
    gemm_a4w4_blockscale,
    gemm_a4w4_blockscale_tune,
    gemm_a4w4o4,
    gemm_a4w4o8,
    gemm_mxfp4_asm,
    gemm_nvfp4_asm,
    unpack_mxfp8_out_scale,
)
from .batched_gemm_op_bf16 import batched_gemm_bf16, batched_gemm_bf16_CK, batched_gemm_bf16_tune  # noqa: E402,F401
from .gemm_op_a8w4 import gemm_a8w4_mxfp8  # noqa: E402,F401
from .gemm_op_a8w8 import (  # noqa: E402,F401
    flatmm_a8w8_blockscale_asm,
    gemm_a8w8_blockscale,
    gemm_a8w8_blockscale_bpreshuffle,
    gemm_a8w8_blockscale_bpreshuffle_asm,
    gemm_a8w8_blockscale_bpreshuffle_cktile,
    gemm_a8w8_blockscale_cktile,
    gemm_a8w8_mxfp8,
    gemm_a8w8_mxfp8_noalloc,
)
from .gemm_op_a16w16 import gemm_a16w16_asm, gemm_a16w16_opus, opus_gemm, opus_gemm_a16w16_tune  # noqa: E402,F401
from .quant import (  # noqa: E402,F401
    dynamic_per_group_scaled_quant,
    get_hip_quant,
    get_torch_quant,
    per_1x32_f4_quant,
    per_1x32_f4_quant_hip,
    per_1x32_f8_scale_f8_quant,
    per_1x32_mx_quant_hip,
)
from .shuffle import (  # noqa: E402,F401
    shuffle_mxfp8fp4_a,
    shuffle_mxfp8fp4_b,
    shuffle_mxfp8fp4_scale,
    shuffle_scale,
    shuffle_scale_f4,
    shuffle_weight,
    shuffle_weight_f4,
)
from .tuned_gemm import TunedGemm, gemm_a16w16, tgemm  # noqa: E402,F401
from . import torch_ops  # noqa: E402,F401  (registers torch.ops.aiter.* with fake-tensor implementations)
