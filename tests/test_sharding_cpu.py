"""Multi-GPU path on CPU: two gloo ranks build their shards with the reader partitioning rule
(shard i of S owns [floor(N*i/S), floor(N*(i+1)/S)), rocAL/source/readers/image/image_reader.cpp:48-67);
the shards are disjoint, cover the dataset, and no data-path collective is involved."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, total, out_dir):
    sys.path.insert(0, ROOT)
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = bench.shard_range(total, rank, world)
    bench.BATCH = total // world
    bench.H_RANGE = (40, 64)
    bench.W_RANGE = (40, 64)
    arena, t = bench.make_shard(rank, world)
    assert len(t) == hi - lo
    # plumbing only: gather the ranges to check the partition, and the max-over-ranks reduction bench.py uses
    ranges = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(ranges, torch.tensor([lo, hi], dtype=torch.int64))
    tm = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    assert float(tm) == float(world)
    np.save(os.path.join(out_dir, "r%d.npy" % rank), np.array([[int(r[0]), int(r[1])] for r in ranges]))
    np.save(os.path.join(out_dir, "sum%d.npy" % rank), np.array([int(arena.astype(np.uint64).sum()), len(t)]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding(tmp_path):
    world, total = 2, 24
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, total, str(tmp_path)), nprocs=world, join=True)
    r = np.load(tmp_path / "r0.npy")
    assert r.tolist() == [[0, 12], [12, 24]]
    s0, s1 = np.load(tmp_path / "sum0.npy"), np.load(tmp_path / "sum1.npy")
    assert s0[1] + s1[1] == total and s0[0] != s1[0]      # different images on the two ranks


def test_shard_range_covers_uneven_datasets():
    sys.path.insert(0, ROOT)
    import bench
    for total in (1, 7, 1000, 1025):
        for shards in (1, 2, 3, 4, 8):
            edges = [bench.shard_range(total, i, shards) for i in range(shards)]
            assert edges[0][0] == 0 and edges[-1][1] == total
            for a, b in zip(edges[:-1], edges[1:]):
                assert a[1] == b[0]
