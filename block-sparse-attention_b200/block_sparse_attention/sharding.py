"""(batch, head) sharding of a block-sparse attention problem over the GPUs of one box.

Every (batch, kv-head group) is independent in forward, backward, quantisation and index construction,
so ranks own disjoint slices and the hot path needs no collective; a gather of the outputs is used for
validation only.  Slices are contiguous in the flattened (batch, kv head) order; when per-slice work is
skewed (``weights``), slices are dealt largest-first to the least-loaded rank instead.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple


def flat_slices(batch: int, kv_heads: int) -> List[Tuple[int, int]]:
    return [(b, h) for b in range(batch) for h in range(kv_heads)]


def shard_batch_heads(batch: int, kv_heads: int, world_size: int, rank: int,
                      weights: Optional[Sequence[float]] = None) -> List[Tuple[int, int]]:
    """Returns the (batch, kv_head) pairs owned by ``rank``."""
    assert world_size >= 1 and 0 <= rank < world_size
    items = flat_slices(batch, kv_heads)
    if weights is None:
        n = len(items)
        base, extra = divmod(n, world_size)
        start = rank * base + min(rank, extra)
        return items[start:start + base + (1 if rank < extra else 0)]
    assert len(weights) == len(items)
    order = sorted(range(len(items)), key=lambda i: (-weights[i], i))
    loads = [0.0] * world_size
    owner = [0] * len(items)
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        owner[i] = r
        loads[r] += weights[i]
    return [items[i] for i in range(len(items)) if owner[i] == rank]
