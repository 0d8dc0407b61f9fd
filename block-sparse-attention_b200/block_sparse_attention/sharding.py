"""(batch, head) sharding of a block-sparse attention problem over the GPUs of one box.

Every (batch, kv-head group) is independent in forward, backward, quantisation and index construction,
so ranks own disjoint slices and the hot path needs no collective; a gather of the outputs is used for
validation only.  Slices are contiguous in the flattened (batch, kv head) order; when per-slice work is
skewed (``weights``), slices are dealt largest-first to the least-loaded rank instead.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch


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


def gather_slices(t: torch.Tensor, slices: Sequence[Tuple[int, int]]) -> torch.Tensor:
    """``[B, H, ...]`` -> ``[1, len(slices), ...]``: the (batch, head) slices of one rank as one MHA problem of batch 1."""
    return torch.stack([t[b, h] for b, h in slices]).unsqueeze(0)


def sharded_fwd_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dout: torch.Tensor,
                    q2k_block_index: torch.Tensor, block_sparse_num: int, slices: Sequence[Tuple[int, int]],
                    sparse_block_size: int = 128, buffers: Optional[Dict[str, torch.Tensor]] = None
                    ) -> Dict[str, torch.Tensor]:
    """Forward + backward of the slices a rank owns (MHA, fixed block count): the slices are gathered into one
    ``[1, n, S, D]`` problem, which the kernels treat exactly like n heads of one batch, so every slice comes out
    bit-identical to the same slice of the unsharded call.  ``q, k, v, dout`` are either the whole ``[B, H, S, D]``
    tensors or, with ``buffers`` (the gathered inputs prepared once by the caller), ignored.  Returns
    ``out, lse, dq, dk, dv`` of shape ``[1, n, ...]`` in the order of ``slices``."""
    from .bsa_attn_interface import bsa_attn_bwd, bsa_attn_fwd
    if buffers is None:
        buffers = {"q": gather_slices(q, slices), "k": gather_slices(k, slices), "v": gather_slices(v, slices),
                   "dout": gather_slices(dout, slices), "index": gather_slices(q2k_block_index, slices).contiguous()}
    b = buffers
    out, lse = bsa_attn_fwd(b["q"], b["k"], b["v"], b["index"], block_sparse_num, return_lse=True,
                            out=b.get("out"), lse=b.get("lse"), sparse_block_size=sparse_block_size)
    dq, dk, dv = bsa_attn_bwd(b["dout"], b["q"], b["k"], b["v"], out, lse, b["index"], block_sparse_num,
                              dq=b.get("dq"), dk=b.get("dk"), dv=b.get("dv"), sparse_block_size=sparse_block_size)
    return {"out": out, "lse": lse, "dq": dq, "dk": dk, "dv": dv}
