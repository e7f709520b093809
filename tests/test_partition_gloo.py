"""The N > 1 path on the CPU: two gloo ranks partition the pair sweep and a sharded batch the way
bench.py does on GPUs (no collective on the data path; results gathered on the host)."""
import os
import sys

import pytest
import torch.multiprocessing as mp

from bfuse_project_b200 import partition

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["cfg1", "cfg3", "cfg4a", "cfg4b", "cfg4c", "cfg5"]


def test_partition_rules():
    for world in (1, 2, 4, 8):
        got = [partition.assign_pairs(NAMES, world, r) for r in range(world)]
        assert sorted(sum(got, [])) == sorted(NAMES)
        shards = [partition.shard_batch(256, world, r) for r in range(world)]
        assert sum(c for _, c in shards) == 256 and shards[0][0] == 0
        assert all(shards[i][0] + shards[i][1] == shards[i + 1][0] for i in range(world - 1))
    assert [partition.shard_batch(10, 4, r) for r in range(4)] == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert partition.shard_batch(0, 2, 1) == (0, 0)
    with pytest.raises(ValueError):
        partition.assign_pairs(NAMES, 2, 2)
    with pytest.raises(ValueError):
        partition.merge_results([{"a": 1}, {"a": 2}])


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = partition.assign_pairs(NAMES, world, rank)
    first, count = partition.shard_batch(256, world, rank)
    # stand-in measurement: a time that depends on the rank, and the shard this rank would process
    results = {n: {"rank": rank, "us": 10.0 + rank} for n in mine}
    gathered = [None] * world
    dist.all_gather_object(gathered, results)
    t = torch.tensor([100.0 + 5.0 * rank])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)          # job time of the sharded workload = slowest rank
    shard = torch.zeros(256, dtype=torch.int32)
    shard[first:first + count] = 1
    dist.all_reduce(shard)                               # test-only: every image is covered exactly once
    if rank == 0:
        merged = partition.merge_results(gathered)
        assert sorted(merged) == sorted(NAMES)
        assert all(merged[n]["rank"] == i % world for i, n in enumerate(NAMES))
        assert float(t) == 100.0 + 5.0 * (world - 1)
        assert int(shard.min()) == 1 and int(shard.max()) == 1
        open(os.path.join(out_dir, "ok"), "w").write("ok")
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_partition_and_gather(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()
