"""GPU parity of the backward pass (BF16, MHA, D = 128, 128- and 64-token blocks) against torch autograd on
the CPU oracle.  Tolerance per gradient is the reference's: 3 * |bf16 autograd - fp32 autograd|max +
3 * bf16 round-trip eps + 5e-3 (tests/test_flash_bwd.py:53-61)."""
import math

import pytest
import torch

from helpers import bf16_from_bits, bf16_roundtrip_eps, load_golden
from oracle import bsa_oracle as orc

pytestmark = pytest.mark.gpu


def _run(q, k, v, do, index, count, nums=None, scale=None, layout="bhsd", bucket=None, bufs=False, blk=128,
         sizes=None):
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd
    c = lambda t: None if t is None else t.cuda()
    qc, kc, vc, doc, ic, nc, sc = c(q), c(k), c(v), c(do), c(index), c(nums), c(sizes)
    if layout == "bshd":
        qc, kc, vc, doc = (t.transpose(1, 2).contiguous() for t in (qc, kc, vc, doc))
    out, lse = bsa_attn_fwd(qc, kc, vc, ic, count, block_sizes=sc, q2k_block_nums=nc, softmax_scale=scale,
                            return_lse=True, layout=layout, sparse_block_size=blk,
                            allow_empty_block_nums=True)
    kw = {}
    if bufs:
        kw = dict(dq=torch.full_like(qc, 7.0), dk=torch.full_like(kc, 7.0), dv=torch.full_like(vc, 7.0))
    dq, dk, dv = bsa_attn_bwd(doc, qc, kc, vc, out, lse, ic, count, block_sizes=sc, q2k_block_nums=nc,
                              softmax_scale=scale, bucket_size_blocks=bucket, layout=layout, sparse_block_size=blk,
                              **kw)
    if bufs:
        assert dq is kw["dq"] and dk is kw["dk"] and dv is kw["dv"]
    if layout == "bshd":
        dq, dk, dv = (t.transpose(1, 2) for t in (dq, dk, dv))
    return dq.float().cpu(), dk.float().cpu(), dv.float().cpu()


def _check(got, q, k, v, do, bias, scale):
    # Rows that attend nothing make the dense autograd reference NaN everywhere (softmax of an all -inf
    # row).  Such rows contribute nothing to any gradient, so for the reference they are given one
    # arbitrary column and a zero upstream gradient, which yields exactly that.
    empty = torch.isinf(bias).all(dim=-1)
    if empty.any():
        bias = bias.clone()
        do = do.clone()
        bias[..., 0] = torch.where(empty, torch.zeros_like(bias[..., 0]), bias[..., 0])
        do[empty] = 0
    _, _, *ref = orc.backward_dense(q, k, v, do, bias, scale, upcast=True)
    _, _, *pt = orc.backward_dense(q, k, v, do, bias, scale, upcast=False)
    for name, g, r, p in zip(("dq", "dk", "dv"), got, ref, pt):
        r = torch.nan_to_num(r.float(), nan=0.0, posinf=0.0, neginf=0.0)
        p = torch.nan_to_num(p.float(), nan=0.0, posinf=0.0, neginf=0.0)
        tol = 3 * (p - r).abs().max().item() + 3 * bf16_roundtrip_eps(r) + 5e-3
        err = (g - r).abs().max().item()
        assert torch.isfinite(g).all(), name
        assert err <= tol, f"{name}: max err {err} > tol {tol}"


def test_golden_backward():
    g = load_golden("bwd_dense.npz")
    q, k, v, do = (bf16_from_bits(g[n]) for n in ("q", "k", "v", "dout"))
    index = torch.from_numpy(g["index"])
    got = _run(q, k, v, do, index, 2)
    for name, t in zip(("dq", "dk", "dv"), got):
        ref = torch.from_numpy(g[name])
        assert (t - ref).abs().max().item() < 3e-2, name
    S = q.shape[2]
    bias = orc.block_sparse_to_attn_bias(index, 2, torch.full((3,), 128, dtype=torch.int32), S, S)
    _check(got, q, k, v, do, bias, 1 / math.sqrt(128))


def _case(seed, B, H, Sq, Sk, counts, poison=True, blk=128):
    gen = torch.Generator().manual_seed(seed)
    q, do = (torch.randn(B, H, Sq, 128, generator=gen).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, H, Sk, 128, generator=gen).bfloat16() for _ in range(2))
    Nq, Nkv = math.ceil(Sq / blk), math.ceil(Sk / blk)
    index = torch.zeros(B, H, Nq, Nkv, dtype=torch.int32)
    nums = torch.zeros(B, H, Nq, dtype=torch.int32)
    i = 0
    for b in range(B):
        for h in range(H):
            for m in range(Nq):
                n = min(counts[i % len(counts)], Nkv)
                i += 1
                nums[b, h, m] = n
                index[b, h, m] = torch.randperm(Nkv, generator=gen).int()
                if poison:
                    index[b, h, m, n:] = 0x3FFFFFFF
    return q, k, v, do, index, nums


@pytest.mark.parametrize("Sq,Sk,counts", [(512, 512, [2, 4, 1, 3]), (1024, 1280, [0, 1, 2, 3, 4, 7, 8, 9]),
                                          (300, 700, [3, 0, 6]), (128, 2048, [16])])
def test_variable_counts_tails_and_empty_rows(Sq, Sk, counts):
    q, k, v, do, index, nums = _case(1, 1, 2, Sq, Sk, counts)
    got = _run(q, k, v, do, index, 0, nums=nums)
    Nkv = math.ceil(Sk / 128)
    sizes = torch.full((Nkv,), 128, dtype=torch.int32)
    sizes[-1] = Sk - (Nkv - 1) * 128
    clean = index.clamp(max=Nkv - 1)
    bias = orc.block_sparse_to_attn_bias(clean, 0, sizes, Sq, Sk, q2k_block_nums=nums)
    _check(got, q, k, v, do, bias, 1 / math.sqrt(128))
    # kv blocks nobody attends and empty query tiles get exact zeros
    attended = torch.zeros(Nkv, dtype=torch.bool)
    for m in range(index.shape[2]):
        attended[clean[0, 0, m, :int(nums[0, 0, m])].long()] = True
    for j in range(Nkv):
        if not attended[j]:
            assert (got[1][0, 0, j * 128:(j + 1) * 128] == 0).all() and (got[2][0, 0, j * 128:(j + 1) * 128] == 0).all()


def test_fixed_count_multi_bucket_bshd_and_buffers():
    q, k, v, do, index, _ = _case(2, 2, 2, 768, 768, [4], poison=False)
    bias = orc.block_sparse_to_attn_bias(index, 4, torch.full((6,), 128, dtype=torch.int32), 768, 768)
    scale = 0.07
    a = _run(q, k, v, do, index, 4, scale=scale, bucket=2)            # three query groups
    b = _run(q, k, v, do, index, 4, scale=scale, bucket=None, layout="bshd", bufs=True)
    _check(a, q, k, v, do, bias, scale)
    for x, y in zip(a, b):
        assert torch.equal(x, y), "grouping / layout must not change the result"


def test_repeat_calls_are_bit_identical_many_tiles():
    """more work items than SMs in both kernels; deterministic accumulation order."""
    q, k, v, do, index, nums = _case(3, 2, 4, 2048, 2048, [5, 3, 8, 1, 0, 6])
    a = _run(q, k, v, do, index, 0, nums=nums)
    b = _run(q, k, v, do, index, 0, nums=nums)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    gq, gk, gv = orc.backward_gathered(q, k, v, do, index.clamp(max=15), 0, nums=nums, heads=[1], batches=[1])
    for got, ref in zip(a, (gq, gk, gv)):
        assert (got[1, 1] - ref[1, 1]).abs().max().item() < 6e-2


# --------------------------------------------------------------------------------------------------
# 64-token blocks (shapes of the reference's tests/test_flash_bwd.py:611-668 plus ragged ones)
# --------------------------------------------------------------------------------------------------
def test_golden_backward_64_token_blocks_with_block_sizes():
    g = load_golden("bwd_blk64_sizes.npz")
    q, k, v, do = (bf16_from_bits(g[n]) for n in ("q", "k", "v", "dout"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    got = _run(q, k, v, do, index, 0, nums=nums, blk=64, sizes=sizes)
    for name, t in zip(("dq", "dk", "dv"), got):
        assert (t - torch.from_numpy(g[name])).abs().max().item() < 3e-2, name
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, q.shape[2], k.shape[2], 64, 64, q2k_block_nums=nums)
    _check(got, q, k, v, do, bias, 1 / math.sqrt(128))
    # tokens beyond a block's valid size take no part: exact zero dK / dV
    for j, n in enumerate(sizes.tolist()):
        lo, hi = j * 64 + n, min((j + 1) * 64, k.shape[2])
        assert (got[1][:, :, lo:hi] == 0).all() and (got[2][:, :, lo:hi] == 0).all()


@pytest.mark.parametrize("variable", [False, True])
@pytest.mark.parametrize("Sq,Sk", [(64, 256), (128, 512), (256, 1024), (512, 512), (1024, 1024), (300, 700)])
def test_64_token_blocks_sparse(Sq, Sk, variable):
    Nkv = math.ceil(Sk / 64)
    counts = [3, 1, 4, 0, 2, 5, Nkv] if variable else [min(3, Nkv)]
    q, k, v, do, index, nums = _case(5, 2 if Sk <= 512 else 1, 4, Sq, Sk, counts, poison=variable, blk=64)
    sizes = torch.full((Nkv,), 64, dtype=torch.int32)
    sizes[-1] = Sk - (Nkv - 1) * 64
    if variable:
        got = _run(q, k, v, do, index, 0, nums=nums, blk=64, sizes=sizes)
        bias = orc.block_sparse_to_attn_bias(index.clamp(max=Nkv - 1), 0, sizes, Sq, Sk, 64, 64, q2k_block_nums=nums)
    else:
        got = _run(q, k, v, do, index, counts[0], blk=64)  # no block_sizes: the tail is masked regardless
        bias = orc.block_sparse_to_attn_bias(index, counts[0], sizes, Sq, Sk, 64, 64)
    _check(got, q, k, v, do, bias, 1 / math.sqrt(128))


def test_64_token_blocks_grouping_layout_and_per_batch_sizes():
    q, k, v, do, index, nums = _case(6, 2, 2, 512, 768, [5, 2, 7, 3], poison=False, blk=64)
    gen = torch.Generator().manual_seed(60)
    sizes = torch.randint(1, 65, (2, 12), generator=gen, dtype=torch.int32)  # rank 2: (batch, kv blocks)
    a = _run(q, k, v, do, index, 0, nums=nums, blk=64, sizes=sizes, bucket=2)  # four query groups
    b = _run(q, k, v, do, index, 0, nums=nums, blk=64, sizes=sizes, bucket=512, layout="bshd", bufs=True)
    for x, y in zip(a, b):
        assert torch.equal(x, y), "grouping / layout must not change the result"
    for bi in range(2):
        bias = orc.block_sparse_to_attn_bias(index[bi:bi + 1], 0, sizes[bi], 512, 768, 64, 64,
                                             q2k_block_nums=nums[bi:bi + 1])
        _check(tuple(t[bi:bi + 1] for t in a), q[bi:bi + 1], k[bi:bi + 1], v[bi:bi + 1], do[bi:bi + 1], bias,
               1 / math.sqrt(128))


def test_64_token_blocks_many_tiles_repeatable():
    """more work items than SMs in both kernels, odd and even entry counts per KV block."""
    q, k, v, do, index, nums = _case(8, 2, 4, 2048, 2048, [5, 3, 8, 1, 0, 6, 9], blk=64)
    a = _run(q, k, v, do, index, 0, nums=nums, blk=64)
    b = _run(q, k, v, do, index, 0, nums=nums, blk=64)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    gq, gk, gv = orc.backward_gathered(q, k, v, do, index.clamp(max=31), 0, nums=nums, blk=64, heads=[2], batches=[1])
    for got, ref in zip(a, (gq, gk, gv)):
        assert (got[1, 2] - ref[1, 2]).abs().max().item() < 6e-2


def test_128_token_blocks_honour_block_sizes_like_the_forward():
    q, k, v, do, index, nums = _case(9, 1, 2, 384, 512, [2, 3, 1], poison=False)
    sizes = torch.tensor([128, 40, 97, 1], dtype=torch.int32)
    got = _run(q, k, v, do, index, 0, nums=nums, sizes=sizes)
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, 384, 512, q2k_block_nums=nums)
    _check(got, q, k, v, do, bias, 1 / math.sqrt(128))


def test_128_token_blocks_per_head_block_sizes():
    """rank 3 (batch, head, kv blocks), as every forward entry accepts it: each (batch, head) slice masks its own
    tokens, checked slice by slice against the dense reference with that slice's sizes."""
    q, k, v, do, index, nums = _case(13, 2, 2, 384, 512, [2, 3, 1, 4], poison=False)
    gen = torch.Generator().manual_seed(61)
    sizes = torch.randint(1, 129, (2, 2, 4), generator=gen, dtype=torch.int32)
    got = _run(q, k, v, do, index, 0, nums=nums, sizes=sizes)
    for bi in range(2):
        for hi in range(2):
            sl = (slice(bi, bi + 1), slice(hi, hi + 1))
            bias = orc.block_sparse_to_attn_bias(index[sl], 0, sizes[bi, hi], 384, 512, q2k_block_nums=nums[sl])
            _check(tuple(t[sl] for t in got), q[sl], k[sl], v[sl], do[sl], bias, 1 / math.sqrt(128))


def test_head_dimension_64_with_128_token_blocks():
    """D = 64 backward exists on the 128-token path only (bsa_attn_interface.py:3867-3873)."""
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd
    gen = torch.Generator().manual_seed(64)
    B, H, Sq, Sk, D = 1, 3, 300, 520, 64
    q, do = (torch.randn(B, H, Sq, D, generator=gen).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, H, Sk, D, generator=gen).bfloat16() for _ in range(2))
    Nq, Nkv = 3, 5
    index = torch.stack([torch.randperm(Nkv, generator=gen) for _ in range(B * H * Nq)]).int().reshape(B, H, Nq, Nkv)
    nums = torch.tensor([[[2, 0, 5], [1, 3, 4], [5, 5, 1]]], dtype=torch.int32)
    qc, kc, vc, doc, ic, nc = (t.cuda() for t in (q, k, v, do, index, nums))
    out, lse = bsa_attn_fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=128)
    got = bsa_attn_bwd(doc, qc, kc, vc, out, lse, ic, 0, q2k_block_nums=nc, sparse_block_size=128)
    assert got[0].shape == q.shape and got[1].shape == k.shape
    sizes = torch.tensor([128, 128, 128, 128, Sk - 512], dtype=torch.int32)
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, Sq, Sk, q2k_block_nums=nums)
    _check(tuple(t.float().cpu() for t in got), q, k, v, do, bias, 1 / math.sqrt(D))
    with pytest.raises(AssertionError):
        bsa_attn_bwd(doc, qc, kc, vc, out, lse, torch.zeros(B, H, 5, 9, dtype=torch.int32, device="cuda"), 1,
                     sparse_block_size=64)


@pytest.mark.parametrize("blk", [128, 64])
def test_skewed_counts_walk_longest_first(blk):
    """more than two work items per SM with per-row counts: both kernels take the longest-first order
    (query tiles by count, KV blocks by the number of tiles attending them); results must not depend on it."""
    S = 8192 if blk == 128 else 4096
    counts = [1, 2, 1, 64 if blk == 128 else 64, 3, 1, 2, 1, 1, 5]
    q, k, v, do, index, nums = _case(21, 2, 4, S, S, counts, blk=blk)
    assert nums.numel() > 2 * 148
    got = _run(q, k, v, do, index, 0, nums=nums, blk=blk)
    Nkv = S // blk
    gq, gk, gv = orc.backward_gathered(q, k, v, do, index.clamp(max=Nkv - 1), 0, nums=nums, blk=blk, heads=[3],
                                       batches=[1])
    for g, ref in zip(got, (gq, gk, gv)):
        assert torch.isfinite(g).all()
        assert (g[1, 3] - ref[1, 3]).abs().max().item() < 6e-2
    again = _run(q, k, v, do, index, 0, nums=nums, blk=blk)
    for x, y in zip(got, again):
        assert torch.equal(x, y)


def test_argument_errors():
    from block_sparse_attention import bsa_attn_bwd
    x = torch.zeros(1, 2, 128, 128, device="cuda").bfloat16()
    lse = torch.zeros(1, 2, 128, device="cuda")
    idx = torch.zeros(1, 2, 1, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(AssertionError):
        bsa_attn_bwd(x, x, x, x, x, lse, idx, 1, sparse_block_size=32)
    with pytest.raises(AssertionError):
        bsa_attn_bwd(x.half(), x.half(), x.half(), x.half(), x.half(), lse, idx, 1, sparse_block_size=128)
    with pytest.raises(AssertionError):
        bsa_attn_bwd(x, x, x[:, :1], x[:, :1], x, lse, idx, 1, sparse_block_size=128)  # GQA


def test_autograd_function_matches_oracle_gradients():
    from block_sparse_attention import block_sparse_attention
    q, k, v, do, index, nums = _case(7, 1, 2, 512, 640, [3, 1, 4, 2], poison=False)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    out = block_sparse_attention(qc, kc, vc, index.cuda(), 0, q2k_block_nums=nums.cuda())
    out.backward(do.cuda())
    bias = orc.block_sparse_to_attn_bias(index, 0, torch.full((5,), 128, dtype=torch.int32), 512, 640,
                                         q2k_block_nums=nums)
    _check(tuple(t.grad.float().cpu() for t in (qc, kc, vc)), q, k, v, do, bias, 1 / math.sqrt(128))


def test_autograd_function_64_token_blocks():
    from block_sparse_attention import block_sparse_attention
    q, k, v, do, index, nums = _case(12, 1, 2, 256, 320, [3, 1, 4, 2], poison=False, blk=64)
    sizes = torch.tensor([64, 10, 64, 33, 64], dtype=torch.int32)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    out = block_sparse_attention(qc, kc, vc, index.cuda(), 0, q2k_block_nums=nums.cuda(), sparse_block_size=64,
                                 block_sizes=sizes.cuda())
    out.backward(do.cuda())
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, 256, 320, 64, 64, q2k_block_nums=nums)
    _check(tuple(t.grad.float().cpu() for t in (qc, kc, vc)), q, k, v, do, bias, 1 / math.sqrt(128))


def test_custom_op_matches_functional_calls_and_compiles():
    from block_sparse_attention import block_sparse_attention_op, bsa_attn_bwd, bsa_attn_fwd
    q, k, v, do, index, nums = _case(13, 1, 2, 384, 512, [3, 1, 4], poison=False)
    ic, nc, doc = index.cuda(), nums.cuda(), do.cuda()
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    out = block_sparse_attention_op(qc, kc, vc, ic, 0, q2k_block_nums=nc)
    out.backward(doc)
    ref_out, lse = bsa_attn_fwd(qc.detach(), kc.detach(), vc.detach(), ic, 0, q2k_block_nums=nc, return_lse=True,
                                sparse_block_size=128)
    ref = bsa_attn_bwd(doc, qc.detach(), kc.detach(), vc.detach(), ref_out, lse, ic, 0, q2k_block_nums=nc,
                       sparse_block_size=128)
    assert torch.equal(out, ref_out)
    for t, r in zip((qc, kc, vc), ref):
        assert torch.equal(t.grad, r)
    # traced as one opaque node: the graph backend only has to carry the call (no code generation involved)
    fn = torch.compile(lambda a, b, c: block_sparse_attention_op(a, b, c, ic, 0, q2k_block_nums=nc) * 2.0,
                       backend="aot_eager", fullgraph=True)
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (qc, kc, vc))
    out2 = fn(q2, k2, v2)
    out2.backward(doc)
    assert torch.equal(out2, ref_out * 2.0)
    assert torch.allclose(q2.grad.float(), 2 * ref[0].float(), rtol=1e-2, atol=1e-3)
    torch.library.opcheck(torch.ops.bsa_b200.fwd.default,
                          (qc.detach(), kc.detach(), vc.detach(), ic, 0, nc, None, 0.088, 128, "bhsd"),
                          test_utils=("test_schema", "test_faketensor"))


def test_host_pipeline_matches_direct_calls():
    """pinned host tensors in, pinned host tensors out, head chunks pipelined over three streams."""
    from block_sparse_attention import HostPipeline, bsa_attn_bwd, bsa_attn_fwd
    q, k, v, do, index, nums = _case(11, 2, 4, 512, 768, [3, 1, 5, 2, 0, 4], poison=False)
    ic, nc = index.cuda(), nums.cuda()
    host_in = {"q": q.pin_memory(), "k": k.pin_memory(), "v": v.pin_memory(), "dout": do.pin_memory()}
    host_out = {"out": torch.empty_like(q).pin_memory(), "lse": torch.empty(2, 4, 512).pin_memory(),
                "dq": torch.empty_like(q).pin_memory(), "dk": torch.empty_like(k).pin_memory(),
                "dv": torch.empty_like(v).pin_memory()}
    pipe = HostPipeline(2, 4, 512, 768, ic, 0, q2k_block_nums=nc, heads_per_chunk=2)
    pipe.run(host_in, host_out)
    pipe.run(host_in, host_out)  # slots are reused
    torch.cuda.synchronize()
    qc, kc, vc, doc = (t.cuda() for t in (q, k, v, do))
    out, lse = bsa_attn_fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=128)
    dq, dk, dv = bsa_attn_bwd(doc, qc, kc, vc, out, lse, ic, 0, q2k_block_nums=nc, sparse_block_size=128)
    for name, ref in (("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert torch.equal(host_out[name], ref.cpu()), name


def test_backward_passes_launched_one_by_one_give_the_same_gradients():
    """`stages` (a profiling knob of the C entry point): preprocess, dQ and dK/dV launched as three calls write
    exactly what the single call writes."""
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd
    from block_sparse_attention.bsa_attn_interface import _bsa_attn_bwd
    q, k, v, do, index, nums = _case(31, 1, 2, 1024, 1024, [3, 1, 4, 2], blk=128)
    qc, kc, vc, doc, ic, nc = (t.cuda() for t in (q, k, v, do, index, nums))
    out, lse = bsa_attn_fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=128)
    ref = bsa_attn_bwd(doc, qc, kc, vc, out, lse, ic, 0, q2k_block_nums=nc, sparse_block_size=128)
    bufs = [torch.full_like(qc, 3.0) for _ in range(3)]
    for mask in (1, 2, 4):
        _bsa_attn_bwd(doc, qc, kc, vc, out, lse, ic, 0, q2k_block_nums=nc, dq=bufs[0], dk=bufs[1], dv=bufs[2],
                      sparse_block_size=128, stages=mask)
    for a, b in zip(ref, bufs):
        assert torch.equal(a, b)
