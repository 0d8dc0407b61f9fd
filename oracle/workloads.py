"""Seeded synthetic generators for the BASELINE configurations 3, 4 and 5 (sparse metadata only; the
dense tensors are drawn by the caller on the device it wants).  TEST / BENCH INFRASTRUCTURE: imported by
tests/ and bench.py only.  The reference measures on synthetic data as well; nothing here reproduces
items of a public suite.
"""
from __future__ import annotations

import torch


def config3_metadata(seed: int = 0, kv_heads: int = 8, seqlen: int = 65536, group: int = 8, mean_blocks: float = 25.0,
                     empty_fraction: float = 0.02):
    """Packed-GQA blk128 metadata: index [1, kv_heads, tiles, cap], nums [1, kv_heads, tiles].
    Tiles are 128 packed rows (seq*group + head offset); counts ~ Poisson(25) clipped to [0, 512], 2 % of
    the rows forced to 0; every row is a prefix of a random permutation of the KV blocks, so the entries
    beyond the count are valid-but-unused block ids."""
    g = torch.Generator().manual_seed(seed)
    nkv = seqlen // 128
    tiles = seqlen * group // 128
    nums = torch.poisson(torch.full((1, kv_heads, tiles), mean_blocks), generator=g).clamp_(0, min(512, nkv))
    nums = nums.to(torch.int32)
    nums[torch.rand(1, kv_heads, tiles, generator=g) < empty_fraction] = 0
    cap = int(nums.max().item())
    cap = max(2, (cap + 7) // 8 * 8)
    index = torch.empty((1, kv_heads, tiles, cap), dtype=torch.int32)
    for h in range(kv_heads):  # per head to bound the memory of the sort keys
        keys = torch.rand(tiles, nkv, generator=g)
        index[0, h] = keys.argsort(dim=-1)[:, :cap].to(torch.int32)
    return index, nums


def config4_metadata(seed: int = 0, heads: int = 24, blocks: int = 600, band: int = 30, far: int = 60):
    """Video-DiT-like banded pattern for blk128: every query block keeps the KV blocks with |i-j| <= band
    plus `far` distinct random blocks outside the band.  Returns index [1, H, blocks, cap] (ascending),
    nums [1, H, blocks]."""
    g = torch.Generator().manual_seed(seed)
    i = torch.arange(blocks)
    in_band = (i[:, None] - i[None, :]).abs() <= band  # [Nq, Nkv]
    counts = in_band.sum(-1) + far
    cap = int(counts.max())
    index = torch.zeros((1, heads, blocks, cap), dtype=torch.int32)
    nums = counts.to(torch.int32).expand(1, heads, blocks).contiguous()
    for h in range(heads):
        keys = torch.rand(blocks, blocks, generator=g)
        keys[in_band] = 2.0  # never drawn as a far block
        far_ids = keys.argsort(dim=-1)[:, :far]
        sel = in_band.clone()
        sel.scatter_(1, far_ids, True)
        order = torch.where(sel, i[None, :].expand(blocks, blocks), torch.full((1,), blocks + 1)).sort(dim=-1).values
        row = order[:, :cap]
        index[0, h] = torch.where(row > blocks, torch.zeros((), dtype=torch.long), row).to(torch.int32)
    return index, nums


def config5_metadata(seed: int = 0, batch: int = 4, heads: int = 16, blocks: int = 256, heavy_fraction: float = 0.01):
    """blk64 metadata with heavy skew: 1 % of the query-block rows attend all KV blocks, the others 2..8
    blocks including the diagonal.  index [B, H, blocks, blocks] (only the first nums entries are live and
    distinct), nums [B, H, blocks]."""
    g = torch.Generator().manual_seed(seed)
    shape = (batch, heads, blocks)
    nums = torch.randint(2, 9, shape, generator=g, dtype=torch.int32)
    heavy = torch.rand(shape, generator=g) < heavy_fraction
    nums[heavy] = blocks
    index = torch.empty((batch, heads, blocks, blocks), dtype=torch.int32)
    diag = torch.arange(blocks)
    for b in range(batch):
        for h in range(heads):
            keys = torch.rand(blocks, blocks, generator=g)
            keys[diag, diag] = -1.0  # the diagonal block is always first
            index[b, h] = keys.argsort(dim=-1).to(torch.int32)
    return index, nums


def k_with_channel_bias(shape, gen_device_seed: int, device, bias_std: float = 3.0):
    """K ~ N(0,1) + per-channel bias ~ N(0, bias_std): makes the Sage K mean-smoothing matter."""
    g = torch.Generator(device=device).manual_seed(gen_device_seed)
    k = torch.randn(shape, generator=g, device=device)
    bias = torch.randn((1, 1, 1, shape[-1]), generator=g, device=device) * bias_std
    return (k + bias).to(torch.bfloat16)
