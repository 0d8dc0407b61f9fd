"""``torch.library`` registration of the forward / backward as custom operators.

The reference exposes plain Python functions that launch compiled kernels and guards them for fake-tensor
tracing by hand (``is_fake_mode()`` checks throughout bsa_attn_interface.py, e.g. :3430-3445).  Registering
the two operators gives the same drop-in behaviour under ``torch.compile`` / ``torch.export`` without those
guards: ``torch.ops.bsa_b200.fwd`` and ``torch.ops.bsa_b200.bwd`` have fake (shape-only) implementations and
an autograd formula, so a traced graph contains one opaque node per call and the kernels behind the C ABI
run unchanged.  BF16, MHA, D = 128, 64- or 128-token blocks (what the backward kernels are built for).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .bsa_attn_interface import bsa_attn_bwd, bsa_attn_fwd

__all__ = ["block_sparse_attention_op"]


def _lse_shape(q: torch.Tensor, layout: str):
    return (q.shape[0], q.shape[1], q.shape[2]) if layout == "bhsd" else (q.shape[0], q.shape[2], q.shape[1])


@torch.library.custom_op("bsa_b200::fwd", mutates_args=(), device_types="cuda")
def _fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q2k_block_index: torch.Tensor, block_sparse_num: int,
         q2k_block_nums: Optional[torch.Tensor], block_sizes: Optional[torch.Tensor], softmax_scale: float,
         sparse_block_size: int, layout: str) -> Tuple[torch.Tensor, torch.Tensor]:
    out, lse = bsa_attn_fwd(q, k, v, q2k_block_index, block_sparse_num, block_sizes=block_sizes,
                            q2k_block_nums=q2k_block_nums, softmax_scale=softmax_scale, return_lse=True,
                            layout=layout, sparse_block_size=sparse_block_size)
    return out, lse


@_fwd.register_fake
def _fwd_fake(q, k, v, q2k_block_index, block_sparse_num, q2k_block_nums, block_sizes, softmax_scale,
              sparse_block_size, layout):
    return torch.empty_like(q), q.new_empty(_lse_shape(q, layout), dtype=torch.float32)


@torch.library.custom_op("bsa_b200::bwd", mutates_args=(), device_types="cuda")
def _bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
         lse: torch.Tensor, q2k_block_index: torch.Tensor, block_sparse_num: int,
         q2k_block_nums: Optional[torch.Tensor], block_sizes: Optional[torch.Tensor], softmax_scale: float,
         sparse_block_size: int, layout: str) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return bsa_attn_bwd(dout, q, k, v, out, lse, q2k_block_index, block_sparse_num, block_sizes=block_sizes,
                        q2k_block_nums=q2k_block_nums, softmax_scale=softmax_scale, layout=layout,
                        sparse_block_size=sparse_block_size)


@_bwd.register_fake
def _bwd_fake(dout, q, k, v, out, lse, q2k_block_index, block_sparse_num, q2k_block_nums, block_sizes,
              softmax_scale, sparse_block_size, layout):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup_context(ctx, inputs, output):
    q, k, v, index, num, nums, sizes, scale, blk, layout = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, index, nums, sizes)
    ctx.meta = (num, scale, blk, layout)


def _backward(ctx, dout, dlse):
    q, k, v, out, lse, index, nums, sizes = ctx.saved_tensors
    num, scale, blk, layout = ctx.meta
    dq, dk, dv = torch.ops.bsa_b200.bwd(dout.contiguous(), q, k, v, out, lse, index, num, nums, sizes, scale, blk,
                                        layout)
    return dq, dk, dv, None, None, None, None, None, None, None


_fwd.register_autograd(_backward, setup_context=_setup_context)


def block_sparse_attention_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q2k_block_index: torch.Tensor,
                              block_sparse_num: int = 0, q2k_block_nums: Optional[torch.Tensor] = None,
                              block_sizes: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None,
                              sparse_block_size: int = 128, layout: str = "bhsd") -> torch.Tensor:
    """Differentiable, traceable block-sparse attention: one ``torch.ops.bsa_b200.fwd`` node per call."""
    if softmax_scale is None:
        softmax_scale = float(q.shape[-1]) ** -0.5
    return torch.ops.bsa_b200.fwd(q, k, v, q2k_block_index, int(block_sparse_num), q2k_block_nums, block_sizes,
                                  float(softmax_scale), int(sparse_block_size), layout)[0]
