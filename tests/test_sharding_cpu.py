"""Batch sharding, the only multi-GPU scheme of the path: rank r of g owns images
[r*N/g, (r+1)*N/g) as its own dense CHWN tensor, filters are replicated, no exchange step.
Runs two gloo ranks on CPU with the oracle standing in for the device kernel: the shards,
gathered (rank-major) and re-interleaved along the innermost image axis, must equal the
unsharded result bit for bit, and the max-over-ranks reduction used for timing must work."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, shape, out_dir):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import Oracle, _oracle_path
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle = Oracle(_oracle_path())
    N, C, K, H, W = shape
    n_local = N // world
    x = oracle.input_chwn(n_local, C, H, W, seed=0, n_offset=rank * n_local)   # this rank's images only
    g = oracle.filter_crsk(C, K, seed=0)                                       # regenerated, not broadcast
    y = torch.from_numpy(oracle.forward(x, g))
    shards = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(shards, y)                                                 # verification only
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                                   # the timing reduction
    if rank == 0:
        full = torch.cat(shards, dim=3).numpy()                                # image axis is innermost
        np.save(os.path.join(out_dir, "gathered.npy"), full)
        np.save(os.path.join(out_dir, "tmax.npy"), t.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_batch_sharding_matches_unsharded(oracle, tmp_path):
    shape = (64, 16, 64, 7, 7)
    world = 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, shape, str(tmp_path)), nprocs=world, join=True)
    N, C, K, H, W = shape
    x, g = oracle.input_chwn(N, C, H, W, seed=0), oracle.filter_crsk(C, K, seed=0)
    expect = oracle.forward(x, g)
    got = np.load(tmp_path / "gathered.npy")
    assert np.array_equal(got, expect)
    assert float(np.load(tmp_path / "tmax.npy")[0]) == float(world)


def test_shard_sizes_keep_the_tiling_constraint():
    # N = 1024 over 1/2/4/8 ranks stays a multiple of the 32-image tile; 128 per rank is the bench's shard
    for g in (1, 2, 4, 8):
        assert (1024 // g) % 32 == 0
    assert 128 % 32 == 0
