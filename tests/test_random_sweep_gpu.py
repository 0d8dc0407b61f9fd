"""Seeded random sweeps on the GPU against the CPU oracle: shapes, counts and options are drawn at random so that
combinations no hand-written case lists are exercised (ragged tails on both sides, empty rows, every rank of
block_sizes, GQA with and without packing, split-KV, narrow heads, float16).  Tolerances are those of the
hand-written tests: |O| 3e-2, LSE 2e-3, gradients 3 * |bf16 autograd - fp32 autograd| + 3 eps + 5e-3."""
import math
import random

import pytest
import torch

from helpers import bf16_roundtrip_eps
from oracle import bsa_oracle as orc

pytestmark = pytest.mark.gpu


def _cuda(t):
    return None if t is None else t.cuda()


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_forward_random_options(seed):
    from block_sparse_attention import bsa_attn_fwd, check_device_status
    rng = random.Random(seed)
    for case in range(12):
        blk = rng.choice([128, 128, 64])
        Hkv = rng.choice([1, 2])
        G = rng.choice([1, 1, 2, 4, 8]) if blk == 128 else 1  # 64-token blocks are MHA-only, as in the reference
        Hq, B = Hkv * G, rng.choice([1, 2])
        packed = blk == 128 and G > 1 and rng.random() < 0.5
        D = rng.choice([128, 128, 128, 64, 96]) if blk == 128 else 128
        dt = torch.float16 if (blk == 128 and rng.random() < 0.2) else torch.bfloat16
        Sq = max(1, rng.randint(1, 6) * blk - rng.choice([0, 0, 1, 19, blk // 2]))
        Sk = max(1, rng.randint(1, 8) * blk - rng.choice([0, 0, 5, 33, blk // 2]))
        splits = rng.choice([1, 1, 2, 3, "auto"]) if blk == 64 else 1
        gen = torch.Generator().manual_seed(seed * 1000 + case)
        q, k, v = (torch.randn(B, h, s, D, generator=gen).to(dt) for h, s in ((Hq, Sq), (Hkv, Sk), (Hkv, Sk)))
        Hidx = Hkv if packed else Hq
        Nq = math.ceil(Sq * G / blk) if packed else math.ceil(Sq / blk)
        Nkv = math.ceil(Sk / blk)
        cap = rng.randint(1, Nkv)
        nums = torch.randint(0 if rng.random() < 0.3 else 1, cap + 1, (B, Hidx, Nq), generator=gen, dtype=torch.int32)
        index = torch.stack([torch.randperm(Nkv, generator=gen)[:cap] for _ in range(B * Hidx * Nq)])
        index = index.int().reshape(B, Hidx, Nq, cap)
        rank = rng.choice([0, 0, 1, 2, 3])
        sizes = None
        if rank:
            shape = {1: (Nkv,), 2: (B, Nkv), 3: (B, Hkv, Nkv)}[rank]
            sizes = torch.randint(0, blk + 1, shape, generator=gen, dtype=torch.int32)
            sizes[..., -1].clamp_(max=Sk - (Nkv - 1) * blk)
        what = (f"seed {seed} case {case}: blk {blk} B {B} Hq {Hq} Hkv {Hkv} packed {packed} D {D} {dt} Sq {Sq} "
                f"Sk {Sk} cap {cap} splits {splits} block_sizes rank {rank}")
        kw = dict(block_sizes=_cuda(sizes), q2k_block_nums=nums.cuda(), return_lse=True, sparse_block_size=blk,
                  allow_empty_block_nums=True)
        if blk == 128:
            kw["pack_gqa"] = packed
        else:
            kw["kv_splits"] = splits
        out, lse = bsa_attn_fwd(q.cuda(), k.cuda(), v.cuda(), index.cuda(), 0, **kw)
        check_device_status()
        ref = orc.attention_gathered_packed if packed else orc.attention_gathered
        ro, rl = ref(q, k, v, index, 0, nums=nums, sizes=sizes, blk=blk)
        o, l = out.float().cpu(), lse.float().cpu()
        assert torch.isfinite(o).all(), what
        assert (o - ro).abs().max().item() <= 3e-2, what
        fin = torch.isfinite(rl)
        assert torch.equal(l[~fin], rl[~fin]), what  # empty rows: exactly -inf
        if fin.any():
            assert (l[fin] - rl[fin]).abs().max().item() <= 2e-3, what


@pytest.mark.parametrize("seed", [21, 22])
def test_forward_backward_random_shapes(seed):
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd, check_device_status
    rng = random.Random(seed)
    scale = 1.0 / math.sqrt(128)
    for case in range(10):
        blk = rng.choice([128, 128, 64])
        B, H = rng.choice([1, 2]), rng.choice([1, 2, 3])
        Nq, Nkv = rng.randint(1, 7), rng.randint(1, 7)
        Sq = max(1, Nq * blk - rng.choice([0, 0, 1, 17, blk // 2]))
        Sk = max(1, Nkv * blk - rng.choice([0, 0, 3, 40, blk // 2]))
        gen = torch.Generator().manual_seed(seed * 1000 + case)
        q, do = (torch.randn(B, H, Sq, 128, generator=gen).bfloat16() for _ in range(2))
        k, v = (torch.randn(B, H, Sk, 128, generator=gen).bfloat16() for _ in range(2))
        cap = rng.randint(1, Nkv)
        nums = torch.randint(0 if rng.random() < 0.3 else 1, cap + 1, (B, H, Nq), generator=gen, dtype=torch.int32)
        index = torch.stack([torch.randperm(Nkv, generator=gen)[:cap].sort().values for _ in range(B * H * Nq)])
        index = index.int().reshape(B, H, Nq, cap)
        sizes = None
        if rng.random() < 0.4:  # per-(batch, head) valid sizes
            sizes = torch.randint(1, blk + 1, (B, H, Nkv), generator=gen, dtype=torch.int32)
            sizes[..., -1].clamp_(max=Sk - (Nkv - 1) * blk)
        what = f"seed {seed} case {case}: blk {blk} B {B} H {H} Sq {Sq} Sk {Sk} cap {cap} sizes {sizes is not None}"
        out, lse = bsa_attn_fwd(q.cuda(), k.cuda(), v.cuda(), index.cuda(), 0, block_sizes=_cuda(sizes),
                                q2k_block_nums=nums.cuda(), return_lse=True, sparse_block_size=blk,
                                allow_empty_block_nums=True)
        grads = bsa_attn_bwd(do.cuda(), q.cuda(), k.cuda(), v.cuda(), out, lse, index.cuda(), 0,
                             block_sizes=_cuda(sizes), q2k_block_nums=nums.cuda(), sparse_block_size=blk)
        check_device_status()
        bias = torch.full((B, H, Sq, Sk), float("-inf"))
        for b in range(B):
            for h in range(H):
                for m in range(Nq):
                    for e in range(int(nums[b, h, m])):
                        j = int(index[b, h, m, e])
                        n = min(blk, Sk - j * blk) if sizes is None else min(blk, Sk - j * blk, int(sizes[b, h, j]))
                        bias[b, h, m * blk:(m + 1) * blk, j * blk:j * blk + n] = 0.0
        empty = torch.isinf(bias).all(dim=-1)
        ro, _ = orc.attention_dense(q, k, v, bias, scale)
        ro = torch.nan_to_num(ro.float(), nan=0.0)
        o = out.float().cpu()
        assert (o - ro)[~empty].abs().max().item() <= 3e-2 if (~empty).any() else True, what
        assert (o[empty] == 0).all(), what
        if empty.any():  # rows that attend nothing contribute nothing: one arbitrary column, zero upstream gradient
            bias[..., 0] = torch.where(empty, torch.zeros_like(bias[..., 0]), bias[..., 0])
            do = do.clone()
            do[empty] = 0
        _, _, *ref = orc.backward_dense(q, k, v, do, bias, scale, upcast=True)
        _, _, *pt = orc.backward_dense(q, k, v, do, bias, scale, upcast=False)
        for name, g, r, p in zip(("dq", "dk", "dv"), grads, ref, pt):
            r = torch.nan_to_num(r.float(), nan=0.0, posinf=0.0, neginf=0.0)
            p = torch.nan_to_num(p.float(), nan=0.0, posinf=0.0, neginf=0.0)
            tol = 3 * (p - r).abs().max().item() + 3 * bf16_roundtrip_eps(r) + 5e-3
            g = g.float().cpu()
            assert torch.isfinite(g).all(), f"{what}: {name}"
            assert (g - r).abs().max().item() <= tol, f"{what}: {name}"
