"""ctypes binding of libaiter_b200.so.

Mirrors the reference's ctypes caller (aiter/jit/core.py:1457-1553): tensors go in as
`aiter_tensor_t*` (NULL for None), ints as C ints (-1 for None), strings as `const char*`
(NULL for None), bools as ints, floats as floats, and the current CUDA stream is appended as
the trailing `void*`.  A non-zero return raises RuntimeError("<name> failed: <message>").
There is no fallback: if the library is missing the import of this module fails.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .dtypes import aiter_dtype_id

# AITER_B200_LIBRARY points at another build of the library (comparing two builds on one machine)
LIB_PATH = os.environ.get("AITER_B200_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "libaiter_b200.so")


class aiter_tensor_t(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("numel_", ctypes.c_size_t),
        ("ndim", ctypes.c_int),
        ("shape", ctypes.c_int64 * 8),
        ("strides", ctypes.c_int64 * 8),
        ("dtype_", ctypes.c_int),
        ("device_id", ctypes.c_int),
    ]


assert ctypes.sizeof(aiter_tensor_t) == 160, "aiter_tensor_t layout drifted from include/aiter_b200.h"


def torch_to_aiter(t: torch.Tensor) -> aiter_tensor_t:
    shape, strides = t.shape, t.stride()
    ndim = len(shape)
    assert ndim <= 8, f"aiter_tensor_t supports at most 8 dims, got {ndim}"
    at = aiter_tensor_t()
    at.ptr = t.data_ptr()
    at.numel_ = t.numel()
    at.ndim = ndim
    at.shape[:ndim] = shape
    at.strides[:ndim] = strides
    at.dtype_ = aiter_dtype_id(t.dtype)
    idx = t.device.index
    at.device_id = -1 if (t.device.type != "cuda" or idx is None) else idx
    return at


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python aiter_b200/build.py` (needs nvcc). "
            "aiter_b200 has no CPU or PyTorch fallback."
        )
    return ctypes.CDLL(LIB_PATH)


_lib = _load()
if int(os.getenv("AITER_LOG_MORE", "0")) >= 1:
    import logging as _logging

    _logging.getLogger("aiter").info("loaded %s", LIB_PATH)
_lib.aiter_get_last_error.restype = ctypes.c_char_p
_lib.aiter_b200_kernel_list.restype = ctypes.c_char_p
_lib.aiter_b200_heuristic_name.restype = ctypes.c_char_p
_lib.aiter_b200_launch_count.restype = ctypes.c_ulonglong
assert _lib.aiter_ctypes_abi_version() == 2

T, I, S, F = "tensor", "int", "str", "float"
# name -> argument kinds (the stream is appended automatically)
SIGNATURES = {
    "gemm_a4w4_asm": (T, T, T, T, T, S, T, F, F, I, I),
    "gemm_a4w4_blockscale": (T, T, T, T, T, I, S),
    "gemm_a4w4_blockscale_tune": (T, T, T, T, T, I, I),
    "mxfp8_mxfp8_gemm_asm": (T, T, T, T, T, S, I),
    "mxfp8_mxfp4_gemm_asm": (T, T, T, T, T, S, I),
    "mxfp4_gemm_asm": (T, T, T, T, T, T, S, I),
    "nvfp4_gemm_asm": (T, T, T, T, F, F, T, T, S, I),
    "gemm_a16w16_asm": (T, T, T, T, T, I, S, I),
    "opus_gemm_a16w16_tune": (T, T, T, T, I, I),
    "opus_gemm": (T, T, T, T, T, T, T),
    "batched_gemm_bf16": (T, T, T, T, I),
    "batched_gemm_bf16_tune": (T, T, T, I, I),
    "dynamic_per_group_scaled_quant": (T, T, T, I, I, T, I),
    "gemm_a8w8_blockscale": (T, T, T, T, T, I, S),
    "gemm_a8w8_blockscale_tune": (T, T, T, T, T, I, I),
    "gemm_a8w8_blockscale_bpreshuffle": (T, T, T, T, T, I, S),
    "gemm_a8w8_blockscale_bpreshuffle_tune": (T, T, T, T, T, I, I),
    "gemm_a8w8_blockscale_cktile": (T, T, T, T, T, I, I, S),
    "gemm_a8w8_blockscale_cktile_tune": (T, T, T, T, T, I, I, I),
    "gemm_a8w8_blockscale_bpreshuffle_cktile": (T, T, T, T, T, I, S),
    "gemm_a8w8_blockscale_bpreshuffle_cktile_tune": (T, T, T, T, T, I, I, I),
    "flatmm_a8w8_blockscale_asm": (T, T, T, T, T),
    "gemm_a8w8_blockscale_bpreshuffle_asm": (T, T, T, T, T, T, I, S, I, T),
    "aiter_b200_gemm_a8w8_mxfp8_noalloc": (T, T, T, T, T, I, I),
}
EXPORTS = sorted(
    list(SIGNATURES)
    + ["getPaddedM", "aiter_ctypes_abi_version", "aiter_get_last_error", "aiter_clear_last_error",
       "opus_gemm_workspace_init", "aiter_b200_device_status", "aiter_b200_kernel_list",
       "aiter_b200_heuristic_name", "aiter_b200_launch_count", "aiter_b200_noalloc_status",
       "aiter_b200_debug_wait_control"]
)


def _convert(kind, value, keep):
    if kind == T:
        if value is None:
            return None
        at = torch_to_aiter(value)
        keep.append(at)
        return ctypes.byref(at)
    if kind == I:
        return ctypes.c_int(-1 if value is None else int(value))
    if kind == F:
        return ctypes.c_float(float(value))
    if kind == S:
        return None if value is None else ctypes.c_char_p(str(value).encode())
    raise TypeError(kind)


_FUNCS = {}
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


# AITER_LOG_MORE=2 logs every call that crosses the C ABI with its arguments (tensors as shape / dtype / device), as
# the reference's ctypes caller does (aiter/jit/core.py:1466-1469); 1 logs the library path at load
AITER_LOG_MORE = int(os.getenv("AITER_LOG_MORE", "0"))


def _describe(a):
    if isinstance(a, torch.Tensor):
        return f"Tensor{tuple(a.shape)} {str(a.dtype).replace('torch.', '')} {a.device} stride{tuple(a.stride())}"
    return repr(a)


def call(name: str, *args):
    """Call an entry point on the current CUDA stream of the first tensor's device."""
    kinds = SIGNATURES[name]
    assert len(args) == len(kinds), f"{name} takes {len(kinds)} arguments, got {len(args)}"
    if AITER_LOG_MORE == 2:
        import logging

        logging.getLogger("aiter").info("calling %s(%s)", name, ", ".join(_describe(a) for a in args))
    keep = []
    cargs = [_convert(k, a, keep) for k, a in zip(kinds, args)]
    dev = next((a.device for a in args if isinstance(a, torch.Tensor) and a.is_cuda), None)
    if dev is None:
        stream = 0
    elif _raw_stream is not None:
        stream = _raw_stream(dev.index if dev.index is not None else torch.cuda.current_device())
    else:
        stream = torch.cuda.current_stream(dev).cuda_stream
    fn = _FUNCS.get(name)
    if fn is None:
        fn = _FUNCS[name] = getattr(_lib, name)
    rc = fn(*cargs, ctypes.c_void_p(stream))
    if rc != 0:
        msg = _lib.aiter_get_last_error()
        raise RuntimeError(f"{name} failed: {msg.decode() if msg else 'unknown error'}")


def get_padded_m(M: int, N: int, K: int, gl: int) -> int:
    return int(_lib.getPaddedM(int(M), int(N), int(K), int(gl)))


def device_status(device: int = 0):
    """(code, block, split, iteration) of the last expired in-kernel wait on `device`; zeros = healthy.
    Synchronises the device and clears the record."""
    words = (ctypes.c_uint * 4)()
    rc = _lib.aiter_b200_device_status(int(device), words)
    if rc != 0:
        msg = _lib.aiter_get_last_error()
        raise RuntimeError(f"aiter_b200_device_status failed: {msg.decode() if msg else ''}")
    return tuple(int(w) for w in words)


def noalloc_status(device: int = 0):
    """Same record for the allocation-free entry point, which keeps it in its own fixed array."""
    words = (ctypes.c_uint * 4)()
    rc = _lib.aiter_b200_noalloc_status(int(device), words)
    if rc != 0:
        msg = _lib.aiter_get_last_error()
        raise RuntimeError(f"aiter_b200_noalloc_status failed: {msg.decode() if msg else ''}")
    return tuple(int(w) for w in words)


def debug_wait_control(device: int = 0, limit_ns: int = 1_000_000_000, withhold_scales: bool = False) -> None:
    """Bound of the in-kernel waits on `device` and the switch that makes one producer issue nothing (tests of the
    time-out path).  Call with no arguments to restore the defaults."""
    rc = _lib.aiter_b200_debug_wait_control(int(device), ctypes.c_ulonglong(int(limit_ns)), int(bool(withhold_scales)))
    if rc != 0:
        msg = _lib.aiter_get_last_error()
        raise RuntimeError(f"aiter_b200_debug_wait_control failed: {msg.decode() if msg else ''}")


def kernel_list() -> str:
    return _lib.aiter_b200_kernel_list().decode()


def heuristic_name(kind: int, M: int, N: int, K: int):
    l2 = ctypes.c_int(0)
    name = _lib.aiter_b200_heuristic_name(int(kind), int(M), int(N), int(K), ctypes.byref(l2))
    return name.decode(), int(l2.value)


def launch_count() -> int:
    return int(_lib.aiter_b200_launch_count())
