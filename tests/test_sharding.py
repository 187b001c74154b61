"""Multi-GPU host logic on CPU: world_size-2 gloo processes shard a batch, run a per-rank function
on their slice and all-gather the shards (the only collective on this path)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from docc_b200.sharding import gather_shards, shard, shard_range


def test_shard_ranges_partition_exactly():
    for total in (0, 1, 7, 8, 32, 33, 128):
        for world in (1, 2, 3, 4, 8):
            ranges = [shard_range(total, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)  # every rank builds the same full input, as bench.py does
        x = torch.randn(total, 3, 5)
        local = shard(x, rank, world) * 2.0 + 1.0  # stand-in for the per-rank kernel
        full = gather_shards(local, total)
        ok = torch.equal(full, x * 2.0 + 1.0)
        # gather along a non-leading dim as well
        y = torch.randn(4, total)
        full_y = gather_shards(shard(y, rank, world, dim=1).clone(), total, dim=1)
        ok = ok and torch.equal(full_y, y)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [8, 7])
def test_two_rank_gloo_shard_and_gather(total):
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(results) == {0: True, 1: True}
