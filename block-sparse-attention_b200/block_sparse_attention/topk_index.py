"""Top-k block selection: builds the q2k index that the attention kernels consume.

The reference has no operator for this step; its benchmark builds the index with torch
(tests/bench_cutedsl_performance.py:131-167: pooled scores -> ``torch.topk(sorted=False)`` -> ascending sort ->
int32) and its notes name the recipe used by callers (design/fp8/results.md:635-636: mean-pool, top-k,
complete K-block index layout).  Here the three steps run as CUDA kernels behind the C ABI
(``bsa_block_mean``, ``bsa_pooled_scores``, ``bsa_topk_q2k``); the result is deterministic: among equal scores
the lower block id wins, and every row comes out in ascending id order.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _cabi

__all__ = ["block_mean", "pooled_scores", "topk_q2k", "pooled_topk_q2k"]


def block_mean(x: torch.Tensor, block_size: int) -> torch.Tensor:
    """Mean of every ``block_size`` consecutive tokens of a BHSD bf16 tensor -> fp32 [B, H, ceil(S/block), D]."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4
    if x.stride(-1) != 1 or any(s % 4 for s in x.stride()[:3]) or x.data_ptr() % 8:
        x = x.contiguous()
    B, H, S, D = x.shape
    assert D % 4 == 0, "head dimension must be a multiple of 4"
    out = torch.empty((B, H, (S + block_size - 1) // block_size, D), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.load().bsa_block_mean(x.data_ptr(), _cabi.strides3(x), B, H, S, D, int(block_size),
                                                 out.data_ptr(), _cabi.stream_ptr(x.device)), "bsa_block_mean")
    return out


def pooled_scores(q_mean: torch.Tensor, k_mean: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """scores[b,h,m,j] = scale * <q_mean[b,h,m], k_mean[b,h,j]> in fp32 (summed over d in ascending order)."""
    assert q_mean.is_cuda and q_mean.dtype == k_mean.dtype == torch.float32
    B, H, Nq, D = q_mean.shape
    assert k_mean.shape[:2] == (B, H) and k_mean.shape[3] == D
    Nkv = k_mean.shape[2]
    q_mean, k_mean = q_mean.contiguous(), k_mean.contiguous()
    out = torch.empty((B, H, Nq, Nkv), dtype=torch.float32, device=q_mean.device)
    with torch.cuda.device(q_mean.device):
        _cabi.check(_cabi.load().bsa_pooled_scores(q_mean.data_ptr(), k_mean.data_ptr(), B * H, Nq, Nkv, D,
                                                    float(scale), out.data_ptr(),
                                                    _cabi.stream_ptr(q_mean.device)), "bsa_pooled_scores")
    return out


def topk_q2k(scores: torch.Tensor, topk: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32 q2k index [..., topk]: ids of the ``topk`` largest entries of every row of ``scores`` in ascending
    id order (``torch.topk(scores, topk, sorted=False).indices.sort(-1).values`` whenever the scores of a row
    are distinct; ties go to the lower id)."""
    assert scores.is_cuda and scores.dtype == torch.float32
    Nkv = scores.shape[-1]
    assert 1 <= topk <= Nkv, f"topk={topk} must be in [1, {Nkv}]"
    scores = scores.contiguous()
    rows = scores.numel() // Nkv
    if out is None:
        out = torch.empty((*scores.shape[:-1], topk), dtype=torch.int32, device=scores.device)
    assert out.dtype == torch.int32 and out.is_contiguous() and out.shape[:-1] == scores.shape[:-1]
    cap = out.shape[-1]
    assert cap >= topk
    with torch.cuda.device(scores.device):
        _cabi.check(_cabi.load().bsa_topk_q2k(scores.data_ptr(), rows, Nkv, int(topk), cap, out.data_ptr(),
                                               _cabi.stream_ptr(scores.device)), "bsa_topk_q2k")
    return out


def pooled_topk_q2k(q: torch.Tensor, k: torch.Tensor, block_size: int, topk: int,
                    softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Mean-pool Q and K per block (BHSD bf16, MHA), score every (query block, KV block) pair and keep the
    ``topk`` best KV blocks per query block: returns the int32 q2k index [B, H, num_q_blocks, topk]."""
    assert q.shape[:2] == k.shape[:2] and q.shape[3] == k.shape[3], "pooled selection is per (batch, head): MHA shapes"
    scale = 1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else softmax_scale
    return topk_q2k(pooled_scores(block_mean(q, block_size), block_mean(k, block_size), scale), topk)
