"""Sharding of a library node's independent units over the GPUs of one box.

The nodes on this path shard without any data-path exchange: softmax over rows, conv and the
transformer block over batch, attention over batch x head, batched matmul over batch. Each rank
(one process per GPU) runs the single-GPU kernels on its slice; the only collective is one
all-gather of the output shards (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Tuple


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open range of units owned by ``rank``: contiguous, covers [0, total) exactly once,
    sizes differ by at most one (the first ``total % world`` ranks hold one more)."""
    if world < 1 or not (0 <= rank < world) or total < 0:
        raise ValueError(f"bad shard request total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard(tensor, rank: int, world: int, dim: int = 0):
    """The slice of ``tensor`` along ``dim`` that ``rank`` owns (a view)."""
    begin, end = shard_range(tensor.shape[dim], rank, world)
    return tensor.narrow(dim, begin, end - begin)


def gather_shards(local, total: int, dim: int = 0, group=None):
    """All-gathers per-rank output shards along ``dim`` into the full tensor (in rank order).
    Ragged shards are padded to the largest shard so that one ``all_gather_into_tensor`` serves both cases."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if world == 1:
        return local
    moved = local.movedim(dim, 0).contiguous()
    if total % world == 0:
        out = torch.empty((total,) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        dist.all_gather_into_tensor(out, moved, group=group)
    else:
        # ragged shards: pad every shard to the largest one, gather, drop the padding
        per = -(-total // world)
        padded = torch.zeros((per,) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        padded[: moved.shape[0]] = moved
        buf = torch.empty((world * per,) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        dist.all_gather_into_tensor(buf, padded, group=group)
        parts = []
        for r in range(world):
            b, e = shard_range(total, r, world)
            parts.append(buf[r * per : r * per + (e - b)])
        out = torch.cat(parts, dim=0)
    return out.movedim(0, dim)
