"""torch.autograd glue around the functional forward / backward.

The reference exposes only ``bsa_attn_fwd`` / ``bsa_attn_bwd`` and leaves the wiring to its callers; this
module is that wiring, so the engine drops into a training loop: ``block_sparse_attention(q, k, v, index,
...)`` is differentiable w.r.t. q, k and v (BF16, MHA, D = 128, 64- or 128-token blocks - the shapes the
backward kernels are built for).
"""
from __future__ import annotations

from typing import Optional

import torch

from .bsa_attn_interface import bsa_attn_bwd, bsa_attn_fwd

__all__ = ["BlockSparseAttentionFunction", "block_sparse_attention"]


class BlockSparseAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q2k_block_index, block_sparse_num, q2k_block_nums, softmax_scale, layout,
                bucket_size_blocks, sparse_block_size=128, block_sizes=None):
        with torch.no_grad():
            out, lse = bsa_attn_fwd(q, k, v, q2k_block_index, block_sparse_num, block_sizes=block_sizes,
                                    q2k_block_nums=q2k_block_nums, softmax_scale=softmax_scale, return_lse=True,
                                    layout=layout, sparse_block_size=sparse_block_size)
        none = torch.empty(0, device=q.device)
        ctx.save_for_backward(q, k, v, out, lse, q2k_block_index,
                              q2k_block_nums if q2k_block_nums is not None else none,
                              block_sizes if block_sizes is not None else none)
        ctx.block_sparse_num = block_sparse_num
        ctx.has_nums = q2k_block_nums is not None
        ctx.has_sizes = block_sizes is not None
        ctx.sparse_block_size = sparse_block_size
        ctx.softmax_scale = softmax_scale
        ctx.layout = layout
        ctx.bucket_size_blocks = bucket_size_blocks
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, index, nums, sizes = ctx.saved_tensors
        dq, dk, dv = bsa_attn_bwd(dout.contiguous(), q, k, v, out, lse, index, ctx.block_sparse_num,
                                  block_sizes=sizes if ctx.has_sizes else None,
                                  q2k_block_nums=nums if ctx.has_nums else None, softmax_scale=ctx.softmax_scale,
                                  bucket_size_blocks=ctx.bucket_size_blocks, layout=ctx.layout,
                                  sparse_block_size=ctx.sparse_block_size)
        return dq, dk, dv, None, None, None, None, None, None, None, None


def block_sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q2k_block_index: torch.Tensor,
                           block_sparse_num: int = 0, q2k_block_nums: Optional[torch.Tensor] = None,
                           softmax_scale: Optional[float] = None, layout: str = "bhsd",
                           bucket_size_blocks: Optional[int] = None, sparse_block_size: int = 128,
                           block_sizes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable block-sparse attention with 128- or 64-token blocks (see ``bsa_attn_fwd`` for the
    arguments; ``block_sizes`` of rank 1, or rank 2 with 64-token blocks)."""
    return BlockSparseAttentionFunction.apply(q, k, v, q2k_block_index, block_sparse_num, q2k_block_nums,
                                              softmax_scale, layout, bucket_size_blocks, sparse_block_size,
                                              block_sizes)
