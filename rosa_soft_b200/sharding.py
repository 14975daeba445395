"""Partitioning of the operator's independent units across the GPUs of one node.

The operator has no exchange step: rows of different (batch, head) never interact and the
value gradient only sums over the query heads of one value head (reference
rosa_soft/csrc/cuda/rosa_soft_kernels.cu:511,789).  A rank therefore takes whole
(batch x value-head group) units, whole packed sequences, or whole (stream x head) units, runs
the unmodified operator on its slice, and passes the global coordinates of the slice to the
dropout counter so that the masks equal those of the unsharded run.  No collective is needed
for the computation; callers that want the full tensors back gather them afterwards.
"""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass
from typing import List, Sequence, Tuple

_coordinates = threading.local()


def current_dropout_coordinates() -> Tuple[int, int]:
    """(batch_offset, head_offset) that the public operators record for their backward."""
    return getattr(_coordinates, "value", (0, 0))


@contextlib.contextmanager
def dropout_coordinates(batch_offset: int = 0, head_offset: int = 0):
    """Calls of ``rosa_soft`` / ``rosa_soft_varlen`` made inside this context belong to a shard
    whose first sequence and first query head have these global indices: the backward adds them
    to the dropout counter's batch and head words, so the shard draws the masks of the unsharded
    run (reference convention: rosa_soft/soft_reference.py:394-447).  The offsets are captured
    when the forward runs; the backward may run after the context has been left."""
    if batch_offset < 0 or head_offset < 0:
        raise ValueError("shard offsets must be non-negative")
    previous = current_dropout_coordinates()
    _coordinates.value = (int(batch_offset), int(head_offset))
    try:
        yield
    finally:
        _coordinates.value = previous


@dataclass(frozen=True)
class DenseShard:
    """Contiguous block of (batch, value-head) units owned by one rank."""
    batch_start: int
    batch_stop: int
    value_head_start: int
    value_head_stop: int

    def head_slice(self, group: int) -> slice:
        return slice(self.value_head_start * group, self.value_head_stop * group)

    @property
    def dropout_batch_offset(self) -> int:
        return self.batch_start

    def dropout_head_offset(self, group: int) -> int:
        return self.value_head_start * group


def shard_dense(batch: int, value_heads: int, world: int, rank: int) -> DenseShard:
    """Split batch first; when there are more ranks than batch elements, split the value
    heads of each batch element evenly among `world // batch` ranks."""
    if not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if world <= batch:
        if batch % world:
            raise ValueError("batch must be divisible by the number of ranks")
        per = batch // world
        return DenseShard(rank * per, (rank + 1) * per, 0, value_heads)
    if world % batch:
        raise ValueError("the number of ranks must be a multiple of the batch size")
    ways = world // batch
    if value_heads % ways:
        raise ValueError("value heads must be divisible by ranks per batch element")
    per = value_heads // ways
    b, part = divmod(rank, ways)
    return DenseShard(b, b + 1, part * per, (part + 1) * per)


def balance_sequences(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time assignment of packed sequences to ranks by their quadratic
    cost; a sequence is never split.  Returns, per rank, the sorted sequence ordinals."""
    loads = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for ordinal in sorted(range(len(lengths)), key=lambda s: (-lengths[s], s)):
        rank = min(range(world), key=lambda r: (loads[r], r))
        loads[rank] += lengths[ordinal] * lengths[ordinal]
        owned[rank].append(ordinal)
    return [sorted(o) for o in owned]


def packed_shard_offsets(lengths: Sequence[int], owned: Sequence[int]) -> Tuple[List[int], List[int]]:
    """Offsets and token ranges of one rank's share of a packed batch.  The rank keeps EVERY
    sequence ordinal in its ``cu_seqlens`` (the ones it does not own have length zero), because
    the dropout counter's batch word is the sequence ordinal counting empty sequences
    (reference rosa_soft/soft_reference.py:683-699): the shard then needs no offset at all.
    Returns (cu_seqlens of the shard, [start, stop) token ranges of the owned sequences in the
    full packed batch, in ordinal order)."""
    owned_set = set(owned)
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    cu, ranges = [0], []
    for ordinal, n in enumerate(lengths):
        take = n if ordinal in owned_set else 0
        cu.append(cu[-1] + take)
        if take:
            ranges.append((starts[ordinal], starts[ordinal + 1]))
    return cu, ranges


def max_over_ranks(local_ms: float, group=None) -> float:
    """Device time of the slowest rank (the only communication a sharded run needs)."""
    import torch
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        return local_ms
    t = torch.tensor([local_ms], dtype=torch.float64)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def gather_along(tensor, dim: int, group=None):
    """All-gather equal shards along `dim` (outputs along heads or batch), on request only."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    parts = [torch.empty_like(tensor) for _ in range(world)]
    dist.all_gather(parts, tensor.contiguous(), group=group)
    return torch.cat(parts, dim=dim)
