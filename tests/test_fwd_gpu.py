"""GPU parity of the BF16 forward (through the C ABI via the host mirror) against the CPU oracle.

Tolerances are the reference's own (tests/test_flash_fwd.py:322-323, :388-399):
  max|out - ref| <= 2 * max|out_bf16 - ref| + 2 * bf16 round-trip eps, and max|lse - ref| <= 1e-3 on
finite rows; gathered-reference cases use rtol = atol = 3e-2 on O and 2e-3 on LSE (:573-585); empty rows
must be exactly 0 / -inf.
"""
import math

import pytest
import torch

from helpers import bf16_from_bits, bf16_roundtrip_eps, load_golden
from oracle import bsa_oracle as orc

pytestmark = pytest.mark.gpu


def _fwd(*a, **kw):
    from block_sparse_attention import bsa_attn_fwd
    return bsa_attn_fwd(*a, **kw)


def _cuda(*ts):
    return [None if t is None else t.cuda() for t in ts]


def _check(out, lse, ref_out, ref_lse, q, k, v, bias=None, strict=True):
    out = out.float().cpu()
    assert torch.isfinite(out).all()
    if bias is not None:
        out_pt, _ = orc.attention_dense(q, k, v, bias, upcast=False, reorder_ops=True)
        tol = 2 * (out_pt.float() - ref_out).abs().max().item() + 2 * bf16_roundtrip_eps(ref_out)
    else:
        tol = 3e-2
    err = (out - ref_out).abs().max().item()
    assert err <= tol, f"max |out - ref| = {err} > {tol}"
    if lse is not None:
        lse = lse.cpu()
        assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse)), "-inf pattern of LSE differs"
        fin = torch.isfinite(ref_lse)
        if fin.any():
            lerr = (lse[fin] - ref_lse[fin]).abs().max().item()
            assert lerr <= 1e-3, f"max |lse - ref| = {lerr}"
        empty = ~fin
        if empty.any():
            assert (out[empty] == 0).all(), "empty rows must be exact zeros"


def test_config1_golden():
    """BASELINE config 1 (B=1,H=4,S=1024,D=128, 8x8 blocks, diagonal + 1) against the reference output."""
    g = load_golden("fwd_config1.npz")
    q, k, v, idx, n = orc.config1(seed=0)
    qb, kb, vb = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out, lse = _fwd(*_cuda(qb, kb, vb, idx), n, return_lse=True, sparse_block_size=128)
    bias = orc.block_sparse_to_attn_bias(idx, n, torch.full((8,), 128, dtype=torch.int32), 1024, 1024)
    ref_out, ref_lse = orc.attention_dense(qb.float(), kb.float(), vb.float(), bias)
    _check(out, lse, ref_out, ref_lse, qb, kb, vb, bias)
    # and against the committed reference vector (fp32 inputs there: bf16 input rounding adds ~1e-2)
    assert (out.float().cpu()[:, :, ::8] - torch.from_numpy(g["out_rows"])).abs().max() < 4e-2


@pytest.mark.parametrize("blk", [128, 64])
def test_dense_golden_variable_counts_and_block_sizes(blk):
    g = load_golden(f"fwd_dense_blk{blk}.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    out, lse = _fwd(*_cuda(q, k, v, index), 0, block_sizes=sizes.cuda(), q2k_block_nums=nums.cuda(),
                    return_lse=True, sparse_block_size=blk)
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, q.shape[2], k.shape[2], blk, blk, q2k_block_nums=nums)
    ref_out, ref_lse = orc.attention_dense(q.float(), k.float(), v.float(), bias)
    _check(out, lse, ref_out, ref_lse, q, k, v, bias)
    assert torch.allclose(ref_out, torch.from_numpy(g["out"]), atol=1e-2)


def test_packed_gqa_golden():
    g = load_golden("fwd_packed_gqa.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    out, lse = _fwd(*_cuda(q, k, v, index), 0, block_sizes=sizes.cuda(), q2k_block_nums=nums.cuda(),
                    pack_gqa=True, return_lse=True, sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered_packed(q, k, v, index, 0, nums=nums, sizes=sizes)
    _check(out, lse, ref_out, ref_lse, q, k, v)


def test_gathered_blk64_golden():
    g = load_golden("fwd_gathered_blk64.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    out, lse = _fwd(*_cuda(q, k, v, index), 0, block_sizes=sizes.cuda(), q2k_block_nums=nums.cuda(),
                    return_lse=True, sparse_block_size=64)
    _check(out, lse, torch.from_numpy(g["out"]), torch.from_numpy(g["lse"]), q, k, v)


def _random_case(seed, B, Hq, Hkv, Sq, Sk, blk, counts, poison=False, sizes_rank=0, packed=False):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Sq, 128, generator=gen).bfloat16()
    k = torch.randn(B, Hkv, Sk, 128, generator=gen).bfloat16()
    v = torch.randn(B, Hkv, Sk, 128, generator=gen).bfloat16()
    G = Hq // Hkv
    Hidx = Hkv if packed else Hq
    Nq = math.ceil(Sq * G / blk) if packed else math.ceil(Sq / blk)
    Nkv = math.ceil(Sk / blk)
    cap = Nkv
    index = torch.zeros(B, Hidx, Nq, cap, dtype=torch.int32)
    nums = torch.zeros(B, Hidx, Nq, dtype=torch.int32)
    i = 0
    for b in range(B):
        for h in range(Hidx):
            for m in range(Nq):
                n = min(counts[i % len(counts)], Nkv)
                i += 1
                nums[b, h, m] = n
                index[b, h, m] = torch.randperm(Nkv, generator=gen).int()
                if poison:
                    index[b, h, m, n:] = 0x3FFFFFFF
    sizes = None
    if sizes_rank:
        shape = {1: (Nkv,), 2: (B, Nkv), 3: (B, Hkv, Nkv)}[sizes_rank]
        sizes = torch.randint(0, blk + 1, shape, generator=gen, dtype=torch.int32)
        sizes[..., -1].clamp_(max=Sk - (Nkv - 1) * blk)
    return q, k, v, index, nums, sizes


COUNTS = [0, 1, 2, 3, 4, 7, 8, 9, 15, 16, 17]  # the reference's boundary counts (tests/test_flash_fwd.py:935)


@pytest.mark.parametrize("blk,Sq,Sk", [(128, 2304, 2304), (64, 1152, 1152), (128, 1000, 1000), (64, 65, 1000),
                                       (128, 1, 300), (64, 63, 130)])
def test_boundary_counts_poisoned_index(blk, Sq, Sk):
    """odd / zero counts, live garbage beyond the count, partial Q tiles and KV tails (:732-853, :935)."""
    q, k, v, index, nums, _ = _random_case(3, 1, 2, 2, Sq, Sk, blk, COUNTS, poison=True)
    out, lse = _fwd(*_cuda(q, k, v, index), 0, q2k_block_nums=nums.cuda(), return_lse=True, sparse_block_size=blk)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums, blk=blk)
    _check(out, lse, ref_out, ref_lse, q, k, v)


@pytest.mark.parametrize("blk,rank", [(128, 1), (128, 2), (128, 3), (64, 1), (64, 2), (64, 3)])
def test_block_sizes_including_zero(blk, rank):
    q, k, v, index, nums, sizes = _random_case(5, 2, 2, 2, 512, 640, blk, [3, 5, 1, 2], sizes_rank=rank)
    out, lse = _fwd(*_cuda(q, k, v, index), 0, block_sizes=sizes.cuda(), q2k_block_nums=nums.cuda(),
                    return_lse=True, sparse_block_size=blk)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums, sizes=sizes, blk=blk)
    _check(out, lse, ref_out, ref_lse, q, k, v)


@pytest.mark.parametrize("Hq,Hkv,pack", [(4, 2, False), (4, 2, True), (8, 1, True), (8, 1, False)])
def test_gqa_mqa(Hq, Hkv, pack):
    q, k, v, index, nums, _ = _random_case(7, 1, Hq, Hkv, 384, 512, 128, [2, 4, 1, 3], packed=pack)
    out, lse = _fwd(*_cuda(q, k, v, index), 0, q2k_block_nums=nums.cuda(), pack_gqa=pack, return_lse=True,
                    sparse_block_size=128)
    if pack:
        ref_out, ref_lse = orc.attention_gathered_packed(q, k, v, index, 0, nums=nums)
    else:
        ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums)
    _check(out, lse, ref_out, ref_lse, q, k, v)


def test_fixed_count_bshd_layout_and_supplied_buffers():
    q, k, v, index, _, _ = _random_case(9, 2, 2, 2, 256, 512, 128, [4])
    qc, kc, vc, ic = _cuda(q, k, v, index)
    q_bshd, k_bshd, v_bshd = (t.transpose(1, 2).contiguous() for t in (qc, kc, vc))
    out_buf = torch.empty_like(q_bshd)
    lse_buf = torch.empty(2, 2, 256, dtype=torch.float32, device="cuda")
    out, lse = _fwd(q_bshd, k_bshd, v_bshd, ic, 4, out=out_buf, lse=lse_buf, layout="bshd", sparse_block_size=128)
    assert out is out_buf and lse is lse_buf
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 4)
    _check(out.transpose(1, 2), lse, ref_out, ref_lse, q, k, v)
    # always a 2-tuple; no LSE unless asked for
    o2, l2 = _fwd(qc, kc, vc, ic, 4, sparse_block_size=128)
    assert l2 is None and torch.equal(o2, out.transpose(1, 2))


def test_noncontiguous_views_and_softmax_scale():
    q, k, v, index, nums, _ = _random_case(11, 1, 2, 2, 256, 256, 128, [2, 1])
    qc, kc, vc, ic, nc = _cuda(q, k, v, index, nums)
    big = torch.randn(1, 2, 256, 256, device="cuda").bfloat16()
    big[..., :128] = qc
    q_view = big[..., :128]  # row stride 256
    out, lse = _fwd(q_view, kc, vc, ic, 0, q2k_block_nums=nc, softmax_scale=0.05, return_lse=True,
                    sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums, scale=0.05)
    _check(out, lse, ref_out, ref_lse, q, k, v)


@pytest.mark.parametrize("splits", [2, 4])
def test_split_kv_matches_unsplit_and_repeats_bit_exactly(splits):
    """tests/test_flash_fwd.py:1502-1554 (split vs unsplit within 3e-2 / 2e-3) and :1564-1631 (repeatability)."""
    q, k, v, index, nums, _ = _random_case(13, 1, 2, 2, 256, 2048, 64, [32, 1, 9, 0])
    qc, kc, vc, ic, nc = _cuda(q, k, v, index, nums)
    o1, l1 = _fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=64, kv_splits=1)
    o2, l2 = _fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=64, kv_splits=splits)
    o3, l3 = _fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=64, kv_splits=splits)
    assert torch.equal(o2, o3) and torch.equal(l2, l3)
    assert torch.allclose(o1.float(), o2.float(), atol=3e-2, rtol=3e-2)
    fin = torch.isfinite(l1)
    assert torch.equal(fin, torch.isfinite(l2))
    assert torch.allclose(l1[fin], l2[fin], atol=2e-3, rtol=0)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums, blk=64)
    _check(o2, l2, ref_out, ref_lse, q, k, v)


def test_underflowing_rows_and_large_scores():
    """rows whose early blocks underflow after a later, much larger block (the reference's sync
    regression inputs, tests/test_sm100_blk128_sync.py)."""
    gen = torch.Generator().manual_seed(17)
    S = 1024
    q = torch.randn(1, 1, S, 128, generator=gen).bfloat16()
    k = torch.randn(1, 1, S, 128, generator=gen)
    k[:, :, 512:640] *= 12.0  # one block with huge scores
    k = k.bfloat16()
    v = torch.randn(1, 1, S, 128, generator=gen).bfloat16()
    index = torch.stack([torch.randperm(8, generator=gen) for _ in range(8)]).int().reshape(1, 1, 8, 8)
    out, lse = _fwd(*_cuda(q, k, v, index), 8, return_lse=True, sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 8)
    _check(out, lse, ref_out, ref_lse, q, k, v)


def test_known_answers_uniform_softmax():
    """q = 0: out = mean of the selected V rows, lse = log(#selected tokens) (tests/test_flash_fwd.py:1682-1722)."""
    S = 512
    q = torch.zeros(1, 2, S, 128).bfloat16()
    k = torch.randn(1, 2, S, 128).bfloat16()
    v = torch.full((1, 2, S, 128), 0.5).bfloat16()
    index = torch.tensor([0, 1, 2, 3], dtype=torch.int32).expand(1, 2, 4, 4).contiguous()
    out, lse = _fwd(*_cuda(q, k, v, index), 4, return_lse=True, sparse_block_size=128)
    assert torch.allclose(out.float().cpu(), torch.full((1, 2, S, 128), 0.5), atol=1e-3)
    assert torch.allclose(lse.cpu(), torch.full((1, 2, S), math.log(S)), atol=1e-3)


def test_argument_errors_are_assertion_errors():
    q = torch.zeros(1, 2, 128, 128, device="cuda").bfloat16()
    idx = torch.zeros(1, 2, 1, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(AssertionError):
        _fwd(q, q, q, idx, 2, sparse_block_size=32)
    with pytest.raises(AssertionError):
        _fwd(q, q, q, idx, 2, sparse_block_size=128, kv_splits=2)
    with pytest.raises(AssertionError):
        _fwd(q, q, q, idx, 2, sparse_block_size=64, pack_gqa=True)
    with pytest.raises(AssertionError):
        _fwd(q, q, q, idx.long(), 2, sparse_block_size=128)
    with pytest.raises(AssertionError):
        _fwd(q, q, q, idx, 4, sparse_block_size=128)  # count above the index width


def test_medium_uniform_many_tiles():
    """more tiles than SMs: exercises the persistent loop and barrier phases across tiles."""
    q, k, v, index, nums, _ = _random_case(19, 2, 4, 4, 4096, 4096, 128, [6, 5, 8, 2, 0, 11])
    out, lse = _fwd(*_cuda(q, k, v, index), 0, q2k_block_nums=nums.cuda(), return_lse=True, sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums, heads=[0, 3])
    sel = [0, 3]
    _check(out[:, sel], lse[:, sel], ref_out[:, sel], ref_lse[:, sel], q, k, v)


def test_cuda_graph_capture_on_a_side_stream_bf16_and_fp8():
    """calls are capturable and side-stream safe (tests/test_bsa_fp8_blk128.py:372-397,
    tests/test_sm100_blk128_sync.py:37-63): no host synchronisation, no read-back on the call path."""
    from block_sparse_attention import bsa_fp8_blk128_fwd, quantize_sage_bhsd
    q, k, v, index, nums, _ = _random_case(23, 1, 2, 2, 512, 1024, 128, [3, 8, 0, 5])
    qc, kc, vc, ic, nc = _cuda(q, k, v, index, nums)
    eager_out, eager_lse = _fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=128)
    quant = quantize_sage_bhsd(qc, kc, vc)
    eager_fp8 = bsa_fp8_blk128_fwd(*quant, ic, 0, q2k_block_nums=nc, kv_splits=2)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        _fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=128)  # warm-up on the stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            g_out, g_lse = _fwd(qc, kc, vc, ic, 0, q2k_block_nums=nc, return_lse=True, sparse_block_size=128)
            g_fp8 = bsa_fp8_blk128_fwd(*quant, ic, 0, q2k_block_nums=nc, kv_splits=2)
        g_out.zero_()
        g_fp8.zero_()
        graph.replay()
        graph.replay()
    side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    assert torch.equal(g_out, eager_out) and torch.equal(g_lse, eager_lse)
    assert torch.equal(g_fp8, eager_fp8)


def test_block_sizes_larger_than_the_physical_tail_do_not_unmask_padding():
    """a provided extent beyond the tokens that exist must not attend to padding
    (tests/test_bsa_fp8_blk128.py:178-201)."""
    q, k, v, index, nums, _ = _random_case(29, 1, 2, 2, 256, 1000, 128, [8])
    sizes = torch.full((8,), 128, dtype=torch.int32)  # last block really has 104 tokens
    out, lse = _fwd(*_cuda(q, k, v, index), 0, block_sizes=sizes.cuda(), q2k_block_nums=nums.cuda(), return_lse=True,
                    sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums)
    _check(out, lse, ref_out, ref_lse, q, k, v)


def test_batch_stride_beyond_2_to_the_31_elements():
    """views whose batch stride exceeds 2^31 elements (tests/test_flash_fwd.py:1641-1722): 64-bit strides end to end."""
    B, H, S = 2, 1, 256
    stride_b = (1 << 31) + 4096
    store = torch.empty(stride_b + H * S * 128, dtype=torch.bfloat16, device="cuda")
    gen = torch.Generator().manual_seed(31)
    q = torch.randn(B, H, S, 128, generator=gen).bfloat16()
    k = torch.randn(B, H, S, 128, generator=gen).bfloat16()
    v = torch.randn(B, H, S, 128, generator=gen).bfloat16()
    k_view = store.as_strided((B, H, S, 128), (stride_b, S * 128, 128, 1))
    k_view.copy_(k.cuda())
    index = torch.tensor([[0, 1], [1, 0]], dtype=torch.int32).expand(B, H, 2, 2).contiguous()
    out, lse = _fwd(q.cuda(), k_view, v.cuda(), index.cuda(), 2, return_lse=True, sparse_block_size=128)
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 2)
    _check(out, lse, ref_out, ref_lse, q, k, v)


def test_float16_inputs_128_token_blocks():
    """the 128-block forward also takes IEEE half inputs (bsa_attn_interface.py:3527: 'inputs must be
    float16 or bfloat16'); 64-token blocks stay bf16-only like the reference (:2360-2363)."""
    q, k, v, index, nums, sizes = _random_case(37, 1, 4, 2, 384, 640, 128, [3, 5, 0, 1], sizes_rank=1)
    qh, kh, vh = q.half(), k.half(), v.half()
    out, lse = _fwd(qh.cuda(), kh.cuda(), vh.cuda(), index.cuda(), 0, block_sizes=sizes.cuda(),
                    q2k_block_nums=nums.cuda(), return_lse=True, sparse_block_size=128, pack_gqa=False)
    assert out.dtype == torch.float16
    ref_out, ref_lse = orc.attention_gathered(qh, kh, vh, index, 0, nums=nums, sizes=sizes)
    _check(out, lse, ref_out, ref_lse, qh, kh, vh)
    with pytest.raises(AssertionError):
        _fwd(qh.cuda()[:, :2], kh.cuda(), vh.cuda(), index.cuda()[:, :2, :, :4].contiguous(), 2, sparse_block_size=64)


@pytest.mark.parametrize("D", [64, 96])
def test_head_dimensions_below_128_with_128_token_blocks(D):
    """the reference's 128-token forward also takes 64- and 96-wide heads (bsa_fwd_sm100.py:75-78)."""
    gen = torch.Generator().manual_seed(D)
    B, Hq, Hkv, Sq, Sk = 2, 4, 2, 300, 700
    q = torch.randn(B, Hq, Sq, D, generator=gen).bfloat16()
    k = torch.randn(B, Hkv, Sk, D, generator=gen).bfloat16()
    v = torch.randn(B, Hkv, Sk, D, generator=gen).bfloat16()
    Nq, Nkv = 3, 6
    index = torch.stack([torch.randperm(Nkv, generator=gen) for _ in range(B * Hq * Nq)]).int().reshape(B, Hq, Nq, Nkv)
    nums = torch.randint(0, Nkv + 1, (B, Hq, Nq), generator=gen, dtype=torch.int32)
    out, lse = _fwd(*_cuda(q, k, v, index), 0, q2k_block_nums=nums.cuda(), return_lse=True, sparse_block_size=128,
                    pack_gqa=False)
    assert out.shape == q.shape
    ref_out, ref_lse = orc.attention_gathered(q, k, v, index, 0, nums=nums)
    _check(out, lse, ref_out, ref_lse, q, k, v)
    # BSHD layout with a supplied buffer, fixed count
    qs, ks, vs = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    buf = torch.full(qs.shape, 3.0, dtype=torch.bfloat16, device="cuda")
    out2, _ = _fwd(*_cuda(qs, ks, vs, index), 2, layout="bshd", out=buf, return_lse=True, sparse_block_size=128,
                   pack_gqa=False)
    ref2, _ = orc.attention_gathered(q, k, v, index, 2)
    assert (out2.transpose(1, 2).float().cpu() - ref2).abs().max().item() < 3e-2
    with pytest.raises(AssertionError):
        _fwd(*_cuda(q[:, :2], k, v, index[:, :2].contiguous()), 2, sparse_block_size=64)   # 64-token blocks need D = 128
