"""N-sharded (column-parallel) quantised GEMM across the GPUs of one node.

The weight [N, K] is split on N: rank r owns rows [r*N/world, (r+1)*N/world) with their scales; the
activations are replicated; every rank computes its own [M, N/world] slice of the output with no
communication.  The only collective is the optional all-gather of the bf16 output slices
(`torch.distributed.all_gather_into_tensor`, NCCL over NVLink / NVSwitch), which lands them in a
[world, M, N/world] buffer that `gathered_view` exposes as the logical [M, N] matrix.

The (16,16) weight shuffle works on 16-row blocks and the scale layouts on 32-row groups, so each shard
is shuffled on its own; nothing here depends on how the other ranks lay out their shards.
One process per GPU (torchrun / mp.spawn), as in the reference's multi-GPU tests
(op_tests/multigpu_tests/test_allgather.py:32-90).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int, multiple: int = 32):
    """Rows [lo, hi) of an N-row weight owned by `rank`.  N must split into equal shards that are a multiple
    of `multiple` rows (32 keeps whole scale groups on one rank; 16 is the weight-shuffle block)."""
    if n % world != 0 or (n // world) % multiple != 0:
        raise ValueError(f"N={n} does not split into {world} shards that are multiples of {multiple} rows")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(t: torch.Tensor, rank: int, world: int, multiple: int = 32) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[0], rank, world, multiple)
    return t[lo:hi].contiguous()


@dataclass
class ShardedWeight:
    """One rank's shard of a quantised weight, already in the wire layout its GEMM entry point takes."""
    data: torch.Tensor
    scale: Optional[torch.Tensor]
    n_local: int
    n_global: int
    rank: int
    world: int


def shard_quantised_weight(wq: torch.Tensor, ws: Optional[torch.Tensor], rank: int, world: int,
                           shuffle_data: Callable[[torch.Tensor], torch.Tensor],
                           shuffle_scale: Optional[Callable[[torch.Tensor], torch.Tensor]]) -> ShardedWeight:
    """Slice the un-shuffled quantised weight / scales [N, ...] for `rank`, then apply the layout functions
    (e.g. shuffle_weight + e8m0_shuffle for gemm_a4w4, shuffle_mxfp8fp4_b + shuffle_mxfp8fp4_scale for the
    MXFP8 paths) to the shard alone."""
    n = wq.shape[0]
    data = shuffle_data(shard_rows(wq, rank, world))
    scale = None
    if ws is not None:
        s = shard_rows(ws, rank, world)
        scale = shuffle_scale(s) if shuffle_scale is not None else s
    return ShardedWeight(data, scale, n // world, n, rank, world)


class NShardedGemm:
    """Column-parallel GEMM: `gemm(x, x_scale, weight_shard)` -> [M, N/world] on every rank.

    `gemm` is any of the operator entry points wrapped to the signature (A, A_scale, B, B_scale) -> out,
    for example ``lambda a, sa, b, sb: aiter_b200.gemm_a4w4(a, b, sa, sb)``."""

    def __init__(self, weight: ShardedWeight, gemm: Callable[..., torch.Tensor], group=None):
        self.weight, self.gemm, self.group = weight, gemm, group
        self._gather_buf = None

    def forward(self, x: torch.Tensor, x_scale: Optional[torch.Tensor]) -> torch.Tensor:
        out = self.gemm(x, x_scale, self.weight.data, self.weight.scale)
        assert out.shape[-1] == self.weight.n_local, (out.shape, self.weight.n_local)
        return out

    def all_gather(self, local_out: torch.Tensor) -> torch.Tensor:
        """All ranks' [M, N/world] slices -> the logical [M, N] matrix (a strided view of a
        [world, M, N/world] buffer; call .contiguous() if a dense matrix is needed)."""
        world = self.weight.world
        m, n_local = local_out.shape
        if self._gather_buf is None or self._gather_buf.shape != (world, m, n_local) or self._gather_buf.dtype != local_out.dtype:
            self._gather_buf = torch.empty((world, m, n_local), dtype=local_out.dtype, device=local_out.device)
        if world == 1:
            self._gather_buf[0].copy_(local_out)
        else:
            # gather raw bytes: the payload is opaque to the collective and not every backend knows bf16
            dist.all_gather_into_tensor(self._gather_buf.view(torch.uint8).view(world * m, -1), local_out.contiguous().view(torch.uint8),
                                        group=self.group)
        return gathered_view(self._gather_buf)

    def __call__(self, x, x_scale, gather: bool = False):
        out = self.forward(x, x_scale)
        return self.all_gather(out) if gather else out


def gathered_view(buf: torch.Tensor) -> torch.Tensor:
    """[world, M, N/world] -> [M, N] view with column block r coming from rank r."""
    world, m, n_local = buf.shape
    return buf.permute(1, 0, 2).reshape(m, world * n_local)
