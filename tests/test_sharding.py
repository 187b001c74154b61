"""Multi-GPU host logic on CPU: world_size-2 gloo processes shard a batch, run a per-rank function
on their slice and all-gather the shards (the only collective on this path)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from docc_b200.sharding import GatherPlan, gather_shards, shard, shard_range


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


def test_gather_plan_partitions_every_unit_once():
    for total, world, chunks in ((32, 8, 2), (32, 4, 1), (128, 8, 4), (6, 2, 3)):
        seen = []
        for c in range(chunks):
            for r in range(world):
                b, e = GatherPlan(total, r, world, chunks).units(c)
                seen.extend(range(b, e))
        assert seen == list(range(total))  # chunk-major, rank order inside a chunk: what an in-place all-gather fills
    with pytest.raises(ValueError):
        GatherPlan(10, 0, 4, 1)
    x = torch.arange(24).reshape(12, 2)
    plan = GatherPlan(12, 1, 2, 3)
    assert plan.local_input(x)[:, 0].tolist() == [4, 6, 12, 14, 20, 22]
    assert plan.local_chunk(plan.local_input(x), 1)[:, 0].tolist() == [12, 14]


def _plan_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        total, chunks = 12, 3
        x = torch.randn(total, 4, 5)  # every rank builds the same global input, as bench.py does
        plan = GatherPlan(total, rank, world, chunks)
        local = plan.local_input(x)
        full = torch.full((total, 4, 5), float("nan"))  # the gathered buffer exists before the step
        ptr = full.data_ptr()

        def compute_chunk(c, out_view):
            assert out_view.data_ptr() == plan.out_slice(full, c).data_ptr()  # the kernel writes into the buffer itself
            out_view.copy_(plan.local_chunk(local, c) * 2.0 + 1.0)  # stand-in for the per-rank kernel

        for _ in range(2):  # a second step reuses the same buffer: no allocation inside a step
            plan.run(full, compute_chunk)
        results[rank] = bool(torch.equal(full, x * 2.0 + 1.0)) and full.data_ptr() == ptr
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_in_place_chunked_gather():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_plan_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(results) == {0: True, 1: True}


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
