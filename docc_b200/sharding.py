"""Sharding of a library node's independent units over the GPUs of one box.

The nodes on this path shard without any data-path exchange: softmax over rows, conv and the
transformer block over batch, attention over batch x head, batched matmul over batch. Each rank
(one process per GPU) runs the single-GPU kernels on its slice; the only collective is the
all-gather of the output shards (NCCL over NVLink on GPUs, gloo in the CPU tests).

Two ways to do that gather:

* ``gather_shards``: one call on a finished local output (allocates the gathered tensor; pads ragged shards).
* ``GatherPlan``: the gathered buffer exists before the step, every rank's kernel writes its shard straight into its
  slice of that buffer, and the all-gather runs in place (send buffer = the rank's slice of the receive buffer), on a
  second stream, one chunk of the batch at a time, so that the gather of chunk c overlaps the kernel of chunk c + 1.
  No copy and no allocation happens inside a step.
"""
from __future__ import annotations

from typing import List, Tuple


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


class GatherPlan:
    """Split-and-gather of ``total`` independent units (dimension 0) over ``world`` ranks in ``chunks`` pieces.

    Unit u of the global tensor belongs to chunk ``u // (world * per)``, inside the chunk to rank
    ``(u % (world * per)) // per`` (``per = total // (world * chunks)`` units per rank and chunk), so every chunk of the
    gathered buffer is ``world`` equal, contiguous slices in rank order: exactly the layout an in-place all-gather
    fills. ``total`` must be a multiple of ``world * chunks`` (ragged splits go through ``gather_shards``).
    """

    def __init__(self, total: int, rank: int, world: int, chunks: int = 1):
        if world < 1 or not (0 <= rank < world) or chunks < 1:
            raise ValueError(f"bad plan rank={rank} world={world} chunks={chunks}")
        if total % (world * chunks) != 0:
            raise ValueError(f"{total} units do not split evenly over {world} ranks x {chunks} chunks")
        self.total, self.rank, self.world, self.chunks = total, rank, world, chunks
        self.per = total // (world * chunks)

    def units(self, chunk: int, rank: int | None = None) -> Tuple[int, int]:
        """Half-open range of global units that ``rank`` (default: this rank) owns in ``chunk``."""
        r = self.rank if rank is None else rank
        begin = (chunk * self.world + r) * self.per
        return begin, begin + self.per

    def local_input(self, full_input):
        """This rank's units of a global input tensor, chunk after chunk (a new contiguous tensor: set-up, not step, work)."""
        import torch

        return torch.cat([full_input[slice(*self.units(c))] for c in range(self.chunks)], dim=0)

    def local_chunk(self, local, chunk: int):
        """View of chunk ``chunk`` inside a tensor laid out like ``local_input``."""
        return local[chunk * self.per : (chunk + 1) * self.per]

    def out_slice(self, full_out, chunk: int):
        """This rank's slice of the gathered buffer for ``chunk``: where the rank's kernel writes its output."""
        return full_out[slice(*self.units(chunk))]

    def chunk_region(self, full_out, chunk: int):
        """All ranks' slices of ``chunk``: the receive buffer of that chunk's all-gather."""
        begin = chunk * self.world * self.per
        return full_out[begin : begin + self.world * self.per]

    def gather_chunk(self, full_out, chunk: int, group=None):
        """In-place all-gather of one chunk (every rank has written ``out_slice(full_out, chunk)``)."""
        import torch.distributed as dist

        if self.world == 1:
            return
        dist.all_gather_into_tensor(self.chunk_region(full_out, chunk), self.out_slice(full_out, chunk), group=group)

    def run(self, full_out, compute_chunk, comm_stream=None, group=None) -> List:
        """``compute_chunk(chunk, out_view)`` launches the rank's kernel(s) for one chunk on the current stream, writing into
        ``out_view``. The chunk's gather then runs on ``comm_stream`` (CUDA) behind an event, overlapping the next chunk's
        kernels. Returns the events recorded after each chunk's kernels (empty on CPU). The caller synchronises
        ``comm_stream`` (or waits on it) before reading ``full_out``."""
        import torch

        events = []
        cuda = full_out.is_cuda
        for c in range(self.chunks):
            compute_chunk(c, self.out_slice(full_out, c))
            if cuda and comm_stream is not None and self.world > 1:
                ev = torch.cuda.Event()
                ev.record()
                events.append(ev)
                comm_stream.wait_event(ev)
                with torch.cuda.stream(comm_stream):
                    self.gather_chunk(full_out, c, group)
            else:
                self.gather_chunk(full_out, c, group)
        return events
