"""GPU parity of the top-k index producer (block means, pooled scores, top-k selection) through the C ABI.
Index work is bit-exact; the fp32 means / scores are compared with rtol 1e-5 (different summation order)."""
import math

import pytest
import torch

from helpers import load_golden
from oracle import bsa_oracle as orc

pytestmark = pytest.mark.gpu


def test_golden_recipe_of_the_reference_benchmark():
    from block_sparse_attention import topk_q2k
    g = load_golden("topk_q2k.npz")
    scores, ref = torch.from_numpy(g["scores"]), torch.from_numpy(g["index"])
    got = topk_q2k(scores.cuda(), ref.shape[-1]).cpu()
    assert got.dtype == torch.int32 and torch.equal(got, ref)


@pytest.mark.parametrize("Nkv,k", [(1, 1), (2, 1), (33, 33), (256, 26), (600, 150), (1000, 999), (4096, 342), (8192, 4096)])
def test_selection_sizes_and_padding(Nkv, k):
    from block_sparse_attention import topk_q2k
    gen = torch.Generator().manual_seed(Nkv + k)
    scores = torch.randn(3, 5, Nkv, generator=gen)
    out = torch.full((3, 5, k + 3), -7, dtype=torch.int32, device="cuda")
    got = topk_q2k(scores.cuda(), k, out=out).cpu()
    assert torch.equal(got[..., :k], orc.topk_q2k(scores, k))
    assert (got[..., k:] == -7).all(), "entries beyond k stay untouched"


def test_ties_nan_and_infinities():
    from block_sparse_attention import topk_q2k
    scores = torch.tensor([[1.0, 3.0, 3.0, 3.0, 0.0, 3.0, -1.0, 2.0],
                           [0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0],
                           [float("-inf"), float("inf"), 5.0, float("nan"), -0.0, 0.0, 1e-45, -1e-45]])
    got = topk_q2k(scores.cuda(), 3).cpu()
    assert got[0].tolist() == [1, 2, 3]      # four-way tie: the lower ids win
    assert got[1].tolist() == [0, 1, 2]
    assert got[2].tolist() == [1, 2, 3]      # NaN ranks above +inf, like torch.topk
    assert torch.equal(got[:2], orc.topk_q2k(scores[:2], 3))
    # a NaN with the sign bit set (the default quiet NaN of x86 arithmetic, 0xFFC00000) ranks the same way
    scores = torch.tensor([[2.0, 0.0, float("inf"), 1.0, float("-inf")]])
    scores.view(torch.int32)[0, 1] = 0xFFC00000 - (1 << 32)
    assert torch.isnan(scores[0, 1])
    assert topk_q2k(scores.cuda(), 2).cpu()[0].tolist() == [1, 2]
    assert torch.topk(scores, 2).indices.sort().values[0].tolist() == [1, 2]


def test_block_mean_and_scores_and_end_to_end_index():
    from block_sparse_attention import block_mean, pooled_scores, pooled_topk_q2k, bsa_attn_fwd
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(2, 3, 1000, 128, generator=gen).bfloat16()
    k = torch.randn(2, 3, 1300, 128, generator=gen).bfloat16()
    for blk in (128, 64):
        qm, km = block_mean(q.cuda(), blk), block_mean(k.cuda(), blk)
        assert torch.allclose(qm.cpu(), orc.block_mean(q, blk), rtol=1e-5, atol=1e-6)
        assert torch.allclose(km.cpu(), orc.block_mean(k, blk), rtol=1e-5, atol=1e-6)
        sc = pooled_scores(qm, km, 0.5)
        ref = torch.einsum("bhmd,bhjd->bhmj", qm.cpu().double(), km.cpu().double()).float() * 0.5
        assert torch.allclose(sc.cpu(), ref, rtol=1e-5, atol=1e-6)
        # selection is bit-exact given the same scores
        idx = pooled_topk_q2k(q.cuda(), k.cuda(), blk, 5)
        assert torch.equal(idx.cpu(), orc.topk_q2k(pooled_scores(qm, km, 1 / math.sqrt(128)).cpu(), 5))
    # a strided (BSHD-backed) view gives the same means
    qs = q.transpose(1, 2).contiguous().transpose(1, 2)
    assert torch.equal(block_mean(qs.cuda(), 128), block_mean(q.cuda(), 128))
    # the produced index feeds the attention forward directly
    v = torch.randn(2, 3, 1300, 128, generator=gen).bfloat16()
    idx = pooled_topk_q2k(q.cuda(), k.cuda(), 128, 4)
    out, lse = bsa_attn_fwd(q.cuda(), k.cuda(), v.cuda(), idx, 4, return_lse=True, sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, idx.cpu(), 4)
    assert (out.float().cpu() - ref_out).abs().max() < 3e-2 and (lse.cpu() - ref_lse).abs().max() < 2e-3


def test_argument_errors():
    from block_sparse_attention import topk_q2k
    s = torch.zeros(2, 8, device="cuda")
    with pytest.raises(AssertionError):
        topk_q2k(s, 0)
    with pytest.raises(AssertionError):
        topk_q2k(s, 9)
    with pytest.raises(AssertionError):
        topk_q2k(torch.zeros(1, 8193, device="cuda"), 4)   # more KV blocks per row than the kernel sorts
