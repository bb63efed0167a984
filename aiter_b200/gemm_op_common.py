"""reference: aiter/ops/gemm_op_common.py:7-8."""
from ._ffi import get_padded_m  # noqa: F401
