"""Tuned (M,N,K) -> kernel tables.

Same schema, same environment variables and the same look-up order as the reference
(aiter/jit/core.py:90-139,217-377; aiter/ops/gemm_op_a4w4.py:33-78): each table is a CSV keyed
by (gfx, cu_num, M, N, K[, ...]); `AITER_CONFIG_GEMM_*` may name one file or an os.pathsep-separated
list (rows merged, the lowest `us` wins per key); a shape is looked up as M, then getPaddedM(gl=0),
then getPaddedM(gl=1).  On this hardware the `gfx` column reads "sm_100a" and `cu_num` is the SM count.
A legacy file without a `gfx` column falls back to a cu_num-only key with a warning.
"""
from __future__ import annotations

import csv
import functools
import logging
import os

logger = logging.getLogger("aiter")

THIS_DIR = os.path.dirname(os.path.abspath(__file__))
CONFIG_DIR = os.path.join(THIS_DIR, "configs")
AITER_LOG_TUNED_CONFIG = int(os.getenv("AITER_LOG_TUNED_CONFIG", "0"))

# table name -> (environment variable, default file)
TABLES = {
    "a4w4": ("AITER_CONFIG_GEMM_A4W4", "a4w4_blockscale_tuned_gemm.csv"),
    "a8w8_blockscale": ("AITER_CONFIG_GEMM_A8W8_BLOCKSCALE", "a8w8_blockscale_tuned_gemm.csv"),
    "a8w8_blockscale_bpreshuffle": ("AITER_CONFIG_GEMM_A8W8_BLOCKSCALE_BPRESHUFFLE", "a8w8_blockscale_bpreshuffle_tuned_gemm.csv"),
    "bf16": ("AITER_CONFIG_GEMM_BF16", "bf16_tuned_gemm.csv"),
    "a8w8_mxfp8": ("AITER_CONFIG_GEMM_A8W8_MXFP8", "a8w8_mxfp8_tuned_gemm.csv"),
    "a8w4_mxfp8": ("AITER_CONFIG_GEMM_A8W4_MXFP8", "a8w4_mxfp8_tuned_gemm.csv"),
    "bf16_batched": ("AITER_CONFIG_BF16_BATCHED_GEMM", "bf16_tuned_batched_gemm.csv"),  # keyed (B, M, N, K)
}
SHAPE_KEYS = ("M", "N", "K")
BF16_EXTRA_KEYS = ("bias", "dtype", "outdtype", "scaleAB", "bpreshuffle")
_INT_COLS = {"cu_num", "B", "M", "N", "K", "kernelId", "splitK", "solidx"}
_BOOL_COLS = {"bias", "scaleAB", "bpreshuffle"}


@functools.lru_cache(maxsize=1)
def get_gfx() -> str:
    return os.getenv("GPU_ARCHS", "sm_100a").split(";")[0]


@functools.lru_cache(maxsize=1)
def get_cu_num() -> int:
    env = os.getenv("CU_NUM")
    if env:
        return int(env)
    try:
        import torch

        if torch.cuda.is_available():
            return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    except Exception:  # pragma: no cover - probing only
        pass
    return 148


def config_paths(table: str):
    env, default = TABLES[table]
    value = os.getenv(env)
    if value:
        return [p for p in value.split(os.pathsep) if p]
    return [os.path.join(CONFIG_DIR, default)]


def _parse(col, val):
    if val is None or val == "":
        return None
    if col in _BOOL_COLS:
        return str(val).strip().lower() in ("1", "true")
    if col in _INT_COLS:
        return int(float(val))
    if col in ("us", "tflops", "bw", "errRatio", "err_ratio"):
        try:
            return float(val)
        except ValueError:
            return None
    return val


def read_table(paths, extra_keys=()):
    """-> (dict key -> row, has_gfx).  Missing files are skipped; none existing raises."""
    rows, has_gfx, seen_any = {}, True, False
    for path in paths:
        if not os.path.exists(path):
            logger.info(f"path {path} (not exist)")
            continue
        seen_any = True
        with open(path, newline="") as f:
            reader = csv.DictReader(f)
            file_has_gfx = "gfx" in (reader.fieldnames or [])
            if not file_has_gfx:
                logger.warning(f"{path} has no 'gfx' column -- falling back to cu_num-only key. Re-run the tuner or migrate the CSV.")
                has_gfx = False
            for raw in reader:
                row = {c: _parse(c, v) for c, v in raw.items()}
                key = tuple(row.get(c) for c in (("gfx",) if file_has_gfx else ()) + ("cu_num",) + SHAPE_KEYS + tuple(extra_keys))
                old = rows.get(key)
                if old is None or (row.get("us") is not None and (old.get("us") is None or row["us"] < old["us"])):
                    rows[key] = row
    if not seen_any:
        raise FileNotFoundError(f"No existing config files found in '{os.pathsep.join(paths)}'")
    if not has_gfx:
        # mixed schemas: drop the gfx component everywhere
        rows = {(k[1:] if len(k) == 5 + len(extra_keys) else k): v for k, v in rows.items()}
    return rows, has_gfx


class TunedTable:
    """Lazy, cached view of one table with the reference's three-step M look-up."""

    def __init__(self, table: str, extra_keys=()):
        self.table, self.extra_keys = table, tuple(extra_keys)
        self._rows = None
        self._has_gfx = True
        self._cache = {}

    def clear(self):
        self._rows, self._cache = None, {}

    def _load(self):
        if self._rows is None:
            self._rows, self._has_gfx = read_table(config_paths(self.table), self.extra_keys)

    def lookup(self, M: int, N: int, K: int, *extra):
        ck = (M, N, K) + extra
        if ck in self._cache:
            return self._cache[ck]
        from ._ffi import get_padded_m

        self._load()
        gfx, cu = get_gfx(), get_cu_num()
        found = None
        for gl in (None, 0, 1):
            pm = M if gl is None else get_padded_m(M, N, K, gl)
            key = ((gfx,) if self._has_gfx else ()) + (cu, pm, N, K) + extra
            found = self._rows.get(key)
            if found is not None:
                if AITER_LOG_TUNED_CONFIG:
                    logger.info(
                        f"shape is M:{M}, N:{N}, K:{K}, found padded_M: {pm}, N:{N}, K:{K} is tuned on cu_num = {cu} in "
                        f"{config_paths(self.table)}, kernel name is {found.get('kernelName')}, splitK is {found.get('splitK')}!"
                    )
                break
        else:
            logger.info(f"shape is M:{M}, N:{N}, K:{K}, not found tuned config in {config_paths(self.table)}, will use default config!")
        self._cache[ck] = found
        return found
