"""Forward + backward for activations that live in pinned HOST memory.

The (batch, head) slices of a block-sparse attention problem are independent, so a step whose inputs and
outputs sit on the host can be cut into head chunks and pipelined over three CUDA streams: while chunk c
is being computed, chunk c+1 is copied host->device and the results of chunk c-1 are copied device->host
(PCIe is full duplex).  The step then costs about max(H2D, D2H, compute) instead of their sum.  Nothing
here has a counterpart in the reference, which only takes device tensors; the kernels and the numerics are
exactly those of ``bsa_attn_fwd`` / ``bsa_attn_bwd`` called on each chunk.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .bsa_attn_interface import bsa_attn_bwd, bsa_attn_fwd

__all__ = ["HostPipeline"]


class HostPipeline:
    """Reusable pipeline for one problem shape (BF16, MHA, D = 128, 128-token blocks).

    ``run(host_in, host_out)`` takes pinned BHSD host tensors ``q, k, v, dout`` and writes pinned host
    tensors ``out, lse, dq, dk, dv``; the sparse metadata stays on the device.  Device staging buffers for
    two chunks are allocated once in the constructor.
    """

    def __init__(self, batch: int, heads: int, seqlen_q: int, seqlen_k: int, q2k_block_index: torch.Tensor,
                 block_sparse_num: int, q2k_block_nums: Optional[torch.Tensor] = None, heads_per_chunk: int = 8,
                 softmax_scale: Optional[float] = None, device: Optional[torch.device] = None):
        assert heads % heads_per_chunk == 0, "heads_per_chunk must divide the number of heads"
        self.B, self.H, self.Sq, self.Sk = batch, heads, seqlen_q, seqlen_k
        self.hc = heads_per_chunk
        self.index = q2k_block_index
        self.nums = q2k_block_nums
        self.count = block_sparse_num
        self.scale = softmax_scale
        self.dev = device or q2k_block_index.device
        self.streams = {n: torch.cuda.Stream(self.dev) for n in ("h2d", "compute", "d2h")}
        bf = torch.bfloat16
        mk = lambda s, dt=bf: torch.empty(s, dtype=dt, device=self.dev)
        self.slots = []
        for _ in range(2):
            self.slots.append({
                "q": mk((1, self.hc, seqlen_q, 128)), "k": mk((1, self.hc, seqlen_k, 128)),
                "v": mk((1, self.hc, seqlen_k, 128)), "dout": mk((1, self.hc, seqlen_q, 128)),
                "out": mk((1, self.hc, seqlen_q, 128)), "lse": mk((1, self.hc, seqlen_q), torch.float32),
                "dq": mk((1, self.hc, seqlen_q, 128)), "dk": mk((1, self.hc, seqlen_k, 128)),
                "dv": mk((1, self.hc, seqlen_k, 128)),
                "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "stored": torch.cuda.Event(),
            })
        self.chunks = [(b, h0) for b in range(batch) for h0 in range(0, heads, self.hc)]

    def run(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor]) -> None:
        """Enqueues the whole step; the calling (current) stream waits for its completion."""
        cur = torch.cuda.current_stream(self.dev)
        for s in self.streams.values():
            s.wait_stream(cur)
        h2d, comp, d2h = self.streams["h2d"], self.streams["compute"], self.streams["d2h"]
        for n, (b, h0) in enumerate(self.chunks):
            slot = self.slots[n % 2]
            hs = slice(h0, h0 + self.hc)
            with torch.cuda.stream(h2d):
                if n >= 2:
                    h2d.wait_event(slot["computed"])  # the inputs of the chunk two back have been consumed
                for name in ("q", "k", "v", "dout"):
                    slot[name].copy_(host_in[name][b:b + 1, hs], non_blocking=True)
                slot["loaded"].record(h2d)
            with torch.cuda.stream(comp):
                comp.wait_event(slot["loaded"])
                if n >= 2:
                    comp.wait_event(slot["stored"])  # the outputs of the chunk two back have left the slot
                idx = self.index[b:b + 1, hs]
                nums = None if self.nums is None else self.nums[b:b + 1, hs]
                bsa_attn_fwd(slot["q"], slot["k"], slot["v"], idx, self.count, q2k_block_nums=nums,
                             softmax_scale=self.scale, out=slot["out"], lse=slot["lse"], sparse_block_size=128)
                bsa_attn_bwd(slot["dout"], slot["q"], slot["k"], slot["v"], slot["out"], slot["lse"], idx,
                             self.count, q2k_block_nums=nums, softmax_scale=self.scale, dq=slot["dq"],
                             dk=slot["dk"], dv=slot["dv"], sparse_block_size=128)
                slot["computed"].record(comp)
            with torch.cuda.stream(d2h):
                d2h.wait_event(slot["computed"])
                for name in ("out", "lse", "dq", "dk", "dv"):
                    host_out[name][b:b + 1, hs].copy_(slot[name], non_blocking=True)
                slot["stored"].record(d2h)
        for s in self.streams.values():
            cur.wait_stream(s)
