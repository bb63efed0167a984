"""N-sharded MXFP4 GEMM on two GPUs (one process per GPU, NCCL): every rank's kernel output equals its column
block of the oracle's full product, and the NCCL all-gather assembles the logical [M, N] matrix."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import mx_oracle as ox

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import aiter_b200 as ab
        from aiter_b200.dist import NShardedGemm, shard_quantised_weight

        g = torch.Generator().manual_seed(0)
        M, N, K = 96, 512, 1024
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = torch.randn(N, K, generator=g).to(torch.bfloat16)
        xq, xs = ox.quant_mxfp4(x.float().numpy())
        wq, ws = ox.quant_mxfp4(w.float().numpy())
        full = ox.gemm_a4w4_ref(xq, wq, xs, ws)  # bf16 bits [M, N]

        shard = shard_quantised_weight(torch.from_numpy(wq).to(dev), torch.from_numpy(ws).to(dev), rank, world,
                                       lambda t: ab.shuffle_weight(t, layout=(16, 16)), ab.shuffle_scale)
        layer = NShardedGemm(shard, lambda a, sa, b, sb: ab.gemm_a4w4(a, b, sa, sb))
        a_dev = torch.from_numpy(xq).to(dev)
        sa_dev = ab.shuffle_scale(torch.from_numpy(xs).to(dev))
        lo, hi = rank * N // world, (rank + 1) * N // world
        local = layer(a_dev, sa_dev)
        ref = torch.from_numpy(full.view(np.int16).copy()).view(torch.bfloat16).float()
        assert torch.allclose(local.float().cpu(), ref[:, lo:hi], rtol=1e-2, atol=1e-2)
        gathered = layer(a_dev, sa_dev, gather=True)
        torch.cuda.synchronize()
        assert gathered.shape == (M, N)
        assert torch.allclose(gathered.float().cpu(), ref, rtol=1e-2, atol=1e-2)
        assert ab.device_status(rank) == (0, 0, 0, 0)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_n_sharded_gemm_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
