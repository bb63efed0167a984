"""N-sharding logic on CPU ranks (gloo, world_size 2): shards are shuffled independently, the per-rank
GEMMs (the oracle stands in for the CUDA kernel here) reproduce the unsharded result, and the gathered
view puts every rank's column block in place."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mx_oracle as ox


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import aiter_b200 as ab
        from aiter_b200.dist import NShardedGemm, shard_quantised_weight

        g = torch.Generator().manual_seed(0)
        M, N, K = 24, 128, 256
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = torch.randn(N, K, generator=g).to(torch.bfloat16)
        xq, xs = ox.quant_mxfp4(x.float().numpy())
        wq, ws = ox.quant_mxfp4(w.float().numpy())
        full = ox.gemm_a4w4_ref(xq, wq, xs, ws)

        shard = shard_quantised_weight(torch.from_numpy(wq), torch.from_numpy(ws), rank, world,
                                       lambda t: ab.shuffle_weight(t, layout=(16, 16)), ab.shuffle_scale)
        assert shard.data.shape == (N // world, K // 2) and shard.n_local == N // world
        # the shard, un-shuffled again, is exactly this rank's rows of the full weight
        lo, hi = rank * N // world, (rank + 1) * N // world
        assert np.array_equal(ox.shuffle_weight_16x16(wq[lo:hi]), shard.data.numpy())
        assert np.array_equal(ox.e8m0_shuffle(ws[lo:hi], 0x7F), shard.scale.numpy())

        def cpu_gemm(a, sa, b_shuffled, sb_shuffled):
            # the CPU stand-in for the CUDA kernel: undo the wire layouts, run the oracle
            n_loc, kb = b_shuffled.shape
            b = np.empty((n_loc, kb), dtype=np.uint8)
            nn, kk = np.meshgrid(np.arange(n_loc), np.arange(kb), indexing="ij")
            b[nn, kk] = b_shuffled.numpy().reshape(-1)[ox.tile16_offset(nn, kk, kb)]
            mm, ks = np.meshgrid(np.arange(n_loc), np.arange(K // 32), indexing="ij")
            s = sb_shuffled.numpy().reshape(-1)[ox.e8m0_shuffle_offset(mm, ks, sb_shuffled.shape[1])]
            bits = ox.gemm_a4w4_ref(a, b, sa, s)
            return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)

        layer = NShardedGemm(shard, cpu_gemm)
        local = layer(xq, xs)
        assert ox.mismatch_ratio(full[:, lo:hi], local.view(torch.int16).numpy().view(np.uint16)) == 0.0
        gathered = layer(xq, xs, gather=True)
        assert gathered.shape == (M, N)
        assert ox.mismatch_ratio(full, gathered.contiguous().view(torch.int16).numpy().view(np.uint16)) == 0.0
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_n_sharded_gemm_two_cpu_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_bounds_reject_ragged():
    from aiter_b200.dist import shard_bounds

    assert shard_bounds(57344, 3, 8) == (21504, 28672)
    with pytest.raises(ValueError):
        shard_bounds(100, 0, 8)
