"""Batch sharding and the max-over-ranks timing reduction, on CPU with world_size-2 gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pytorch_winoconv_b200 import sharding


@pytest.mark.parametrize("total,world", [(256, 1), (256, 2), (256, 8), (10, 4), (3, 8), (0, 2)])
def test_shards_partition_the_batch(total, world):
    shards = sharding.all_shards(total, world)
    assert shards[0][0] == 0 and shards[-1][1] == total
    for (a0, a1), (b0, b1) in zip(shards, shards[1:]):
        assert a1 == b0 and a1 - a0 >= b1 - b0 >= 0
    assert max(e - b for b, e in shards) - min(e - b for b, e in shards) <= 1


def test_bad_rank_rejected():
    with pytest.raises(ValueError):
        sharding.shard_bounds(8, 2, 2)
    with pytest.raises(ValueError):
        sharding.aggregate_throughput([1], [0.0])


def test_aggregate_uses_slowest_rank():
    assert sharding.aggregate_throughput([128, 128], [0.5, 1.0]) == 256.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, e = sharding.shard_bounds(7, world, rank)
        elapsed = 0.25 * (rank + 1)
        slow = sharding.max_over_ranks(elapsed)
        units = sharding.sum_over_ranks(e - b)
        dist.barrier()
        out.put((rank, b, e, slow, units))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_reduction():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(r[1], r[2]) for r in res] == [(0, 4), (4, 7)]
    assert all(r[3] == 0.5 and r[4] == 7.0 for r in res)
