"""CPU: the oracle (oracle/bsa_oracle.py) against golden vectors produced by the reference's own
functions (tests/golden/make_golden.py) and against the literal known-answer cases of its tests."""
import hashlib
import math

import numpy as np
import pytest
import torch

from helpers import bf16_from_bits, load_golden
from oracle import bsa_oracle as orc


@pytest.mark.parametrize("blk", [128, 64])
def test_dense_forward_matches_reference(blk):
    g = load_golden(f"fwd_dense_blk{blk}.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    Sq, Sk = q.shape[2], k.shape[2]
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, Sq, Sk, blk, blk, q2k_block_nums=nums)
    if blk == 128:
        assert np.array_equal(torch.isfinite(bias).numpy().astype(np.uint8), g["bias_finite"])
    out, lse = orc.attention_dense(q, k, v, bias)
    assert torch.allclose(out.float(), torch.from_numpy(g["out"]), atol=1e-2, rtol=0)  # reference output is bf16-rounded
    ref_lse = torch.from_numpy(g["lse"])
    assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse))
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse[fin], ref_lse[fin], atol=1e-5, rtol=0)
    # the gathered formulation is the same function
    og, lg = orc.attention_gathered(q, k, v, index, 0, nums=nums, sizes=sizes, blk=blk)
    out32, _ = orc.attention_dense(q.float(), k.float(), v.float(), bias)
    assert torch.allclose(og, out32, atol=2e-5, rtol=0)
    assert torch.allclose(lg[fin], ref_lse[fin], atol=1e-5, rtol=0)
    assert torch.equal(torch.isinf(lg), torch.isinf(ref_lse))


def test_config1_matches_reference():
    g = load_golden("fwd_config1.npz")
    q, k, v, idx, n = orc.config1(seed=0)
    sha = hashlib.sha256(q.numpy().tobytes() + k.numpy().tobytes() + v.numpy().tobytes()
                         + idx.numpy().tobytes()).hexdigest()
    if sha != str(g["input_sha256"]):
        pytest.skip("torch CPU generator differs from the one that made the fixture")
    bias = orc.block_sparse_to_attn_bias(idx, n, torch.full((8,), 128, dtype=torch.int32), 1024, 1024)
    out, lse = orc.attention_dense(q, k, v, bias)
    assert torch.allclose(out[:, :, ::8], torch.from_numpy(g["out_rows"]), atol=2e-6, rtol=0)
    assert torch.allclose(lse, torch.from_numpy(g["lse"]), atol=2e-6, rtol=0)
    og, lg = orc.attention_gathered(q, k, v, idx, n)
    assert torch.allclose(og[:, :, ::8], torch.from_numpy(g["out_rows"]), atol=5e-6, rtol=0)


def test_packed_gqa_matches_reference():
    g = load_golden("fwd_packed_gqa.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    out, lse = orc.attention_gathered_packed(q, k, v, index, 0, nums=nums, sizes=sizes)
    ref_out, ref_lse = torch.from_numpy(g["out"]), torch.from_numpy(g["lse"])
    assert torch.allclose(out, ref_out, atol=1e-2, rtol=0)
    assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse))
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse[fin], ref_lse[fin], atol=1e-5, rtol=0)
    # dense route with the unpacked bias
    Sq, G = q.shape[2], q.shape[1] // k.shape[1]
    nt = index.shape[2]
    bias_kv = orc.block_sparse_to_attn_bias(index, 0, sizes, nt * 128, k.shape[2], 128, 128, q2k_block_nums=nums)
    bias = orc.unpack_gqa_attn_bias(bias_kv, q.shape[1], G, Sq)
    out2, lse2 = orc.attention_dense(q, k, v, bias)
    assert torch.allclose(out2.float(), ref_out, atol=1e-2, rtol=0)
    assert torch.allclose(lse2[fin], ref_lse[fin], atol=1e-5, rtol=0)


def test_gathered_variable_blk64_matches_reference():
    g = load_golden("fwd_gathered_blk64.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    out, lse = orc.attention_gathered(q, k, v, index, 0, nums=nums, sizes=sizes, blk=64)
    assert torch.allclose(out, torch.from_numpy(g["out"]), atol=2e-6, rtol=0)
    ref_lse = torch.from_numpy(g["lse"])
    assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse))
    assert (out[0, 0, :64] == 0).all() and torch.isinf(lse[0, 0, :64]).all()  # empty row: exact 0 / -inf
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse[fin], ref_lse[fin], atol=2e-6, rtol=0)


@pytest.mark.parametrize("name", ["csr_literal_variable.npz", "csr_random_fixed.npz", "csr_topk_1025.npz"])
def test_csr_matches_reference(name):
    g = load_golden(name)
    q2k = torch.from_numpy(g["q2k"])
    nums = torch.from_numpy(g["nums"]) if g["nums"].size else None
    offsets, rows = orc.bucketed_k2q_csr(q2k, int(g["bsn"]), int(g["nkv"]), int(g["bucket"]), nums)
    assert np.array_equal(offsets.numpy(), g["offsets"])
    flat, lens = [], []
    B, H, G, _ = offsets.shape
    for b in range(B):
        for h in range(H):
            for gq in range(G):
                for j in range(int(g["nkv"])):
                    r = sorted(rows[(b, h, gq, j)])
                    flat.extend(r)
                    lens.append(len(r))
    assert np.array_equal(np.array(flat, np.int32), g["rows_flat"])
    assert np.array_equal(np.array(lens, np.int32), g["rows_len"])


def test_fp8_gathered_and_dequantiser_match_reference():
    g = load_golden("fp8_gathered.npz")
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    out = orc.attention_gathered(q, k, v, index, index.shape[-1], nums=nums, sizes=sizes, return_lse=False)
    assert torch.allclose(out, torch.from_numpy(g["out"]), atol=2e-6, rtol=0)
    q8, k8, v8 = (torch.from_numpy(g[n].copy()).view(torch.float8_e4m3fn) for n in ("q8", "k8", "v8"))
    qs, ks, vs = (torch.from_numpy(g[n]) for n in ("qs", "ks", "vs"))
    dq, dk, dv = orc.sage_dequantize(q8, k8, v8, qs, ks, vs)
    for got, name in ((dq, "deq_q"), (dk, "deq_k"), (dv, "deq_v")):
        assert torch.equal(got.view(torch.int16), torch.from_numpy(g[name].copy()))
    # the oracle's quantiser shares the scale formulas of the reference's all-fp32 recipe
    # (tests/test_bsa_fp8_fwd.py:80-100): scales identical, K bytes identical (same centring and division)
    kp = torch.nn.functional.pad(k, (0, 0, 0, 4))
    vp = torch.nn.functional.pad(v, (0, 0, 0, 4))
    oq8, ok8, ov8, oqs, oks, ovs = orc.sage_quantize(q, kp, vp)
    assert torch.equal(oqs, qs) and torch.equal(ovs, vs)
    assert torch.allclose(oks, ks, rtol=2e-6, atol=2e-8)
    assert (ok8.view(torch.uint8) != k8.view(torch.uint8)).float().mean() < 1e-4
    # Q and V differ from that recipe only by the rounding order, i.e. at most one e4m3 bin
    assert (oq8.float() - q8.float()).abs().max() <= 32 and (ov8.float() - v8.float()).abs().max() <= 32


def test_backward_matches_reference():
    g = load_golden("bwd_dense.npz")
    q, k, v, do = (bf16_from_bits(g[n]) for n in ("q", "k", "v", "dout"))
    index = torch.from_numpy(g["index"])
    S = q.shape[2]
    bias = orc.block_sparse_to_attn_bias(index, 2, torch.full((3,), 128, dtype=torch.int32), S, S)
    scale = 1.0 / math.sqrt(128)
    o, lse, dq, dk, dv = orc.backward_dense(q, k, v, do, bias, scale)
    for got, name in ((dq, "dq"), (dk, "dk"), (dv, "dv"), (lse, "lse")):
        assert torch.allclose(got, torch.from_numpy(g[name]), atol=1e-5, rtol=1e-5), name
    gq, gk, gv = orc.backward_gathered(q, k, v, do, index, 2, scale=scale)
    for got, name in ((gq, "dq"), (gk, "dk"), (gv, "dv")):
        assert torch.allclose(got, torch.from_numpy(g[name]), atol=2e-4, rtol=1e-4), name


def test_backward_64_token_blocks_with_block_sizes_matches_reference():
    g = load_golden("bwd_blk64_sizes.npz")
    q, k, v, do = (bf16_from_bits(g[n]) for n in ("q", "k", "v", "dout"))
    index, nums, sizes = (torch.from_numpy(g[n]) for n in ("index", "nums", "sizes"))
    Sq, Sk = q.shape[2], k.shape[2]
    bias = orc.block_sparse_to_attn_bias(index, 0, sizes, Sq, Sk, 64, 64, q2k_block_nums=nums)
    scale = 1.0 / math.sqrt(128)
    o, lse, dq, dk, dv = orc.backward_dense(q, k, v, do, bias, scale)
    for got, name in ((dq, "dq"), (dk, "dk"), (dv, "dv"), (lse, "lse")):
        assert torch.allclose(got, torch.from_numpy(g[name]), atol=1e-5, rtol=1e-5), name
    gq, gk, gv = orc.backward_gathered(q, k, v, do, index, 0, nums=nums, scale=scale, blk=64, sizes=sizes)
    for got, name in ((gq, "dq"), (gk, "dk"), (gv, "dv")):
        assert torch.allclose(got, torch.from_numpy(g[name]), atol=2e-4, rtol=1e-4), name


def test_topk_index_recipe_matches_torch_topk():
    g = load_golden("topk_q2k.npz")
    scores, ref = torch.from_numpy(g["scores"]), torch.from_numpy(g["index"])
    assert torch.equal(orc.topk_q2k(scores, ref.shape[-1]), ref)
    tied = torch.tensor([[1.0, 3.0, 3.0, 3.0, 0.0, 3.0]])
    assert orc.topk_q2k(tied, 3).tolist() == [[1, 2, 3]]
    x = torch.arange(2 * 1 * 5 * 4, dtype=torch.float32).reshape(2, 1, 5, 4).bfloat16()
    m = orc.block_mean(x, 2)
    assert m.shape == (2, 1, 3, 4) and torch.equal(m[0, 0, 2], x[0, 0, 4].float())


def test_split_policy_matches_reference():
    g = load_golden("policy_blk64_splits.npz")
    for c, s in zip(g["counts"].tolist(), g["splits"].tolist()):
        assert orc.blk64_kv_splits_from_count(c) == s
    # tests/test_flash_fwd.py cases of the auto policy: >= 512 query tiles -> 1
    assert orc.blk64_auto_kv_splits(4, 16, 16384, 256) == 1
    assert orc.blk64_auto_kv_splits(1, 1, 64 * 100, 2048) == 8


def test_fp8_split_policy_matches_reference():
    """Grid generated by running the reference's _sm100_blk64_auto_fp8_kv_splits (tests/golden/make_golden.py)."""
    rows = load_golden("policy_fp8_blk64_splits.npz")["rows"].tolist()
    assert len(rows) > 1000
    for kv_blocks, heads, seqlen_q, batch, num_sms, splits in rows:
        assert orc.blk64_auto_fp8_kv_splits(kv_blocks, heads, seqlen_q, batch, num_sms) == splits


def test_analytic_known_answers():
    """Known-answer rows in the style of tests/test_flash_fwd.py:1682-1722: q = 0 gives a uniform
    softmax, so out = mean(v) over the selected tokens and lse = log(number of selected tokens)."""
    S = 256
    q = torch.zeros(1, 1, S, 128)
    k = torch.randn(1, 1, S, 128, generator=torch.Generator().manual_seed(3))
    v = torch.ones(1, 1, S, 128) * 0.5
    index = torch.tensor([[[[0, 1], [1, 0]]]], dtype=torch.int32)
    out, lse = orc.attention_gathered(q, k, v, index, 2)
    assert torch.allclose(out, torch.full_like(out, 0.5), atol=1e-6)
    assert torch.allclose(lse, torch.full_like(lse, math.log(S)), atol=1e-5)
    sizes = torch.tensor([100, 28], dtype=torch.int32)
    out, lse = orc.attention_gathered(q, k, v, index, 2, sizes=sizes)
    assert torch.allclose(lse, torch.full_like(lse, math.log(128)), atol=1e-5)


def test_combine_is_consistent_with_unsplit():
    gen = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 2, 128, 128, generator=gen) for _ in range(3))
    k = torch.randn(1, 2, 512, 128, generator=gen)
    v = torch.randn(1, 2, 512, 128, generator=gen)
    index = torch.tensor([0, 1, 2, 3], dtype=torch.int32).expand(1, 2, 1, 4).contiguous()
    full, lse_full = orc.attention_gathered(q, k, v, index, 4)
    parts, lses = [], []
    for s in range(2):
        o, l = orc.attention_gathered(q, k, v, index[..., 2 * s:2 * s + 2].contiguous(), 2)
        parts.append(o)
        lses.append(l)
    parts.append(torch.zeros_like(parts[0]))
    lses.append(torch.full_like(lses[0], float("-inf")))  # an empty split
    out, lse = orc.combine_partials(torch.stack(parts), torch.stack(lses))
    assert torch.allclose(out, full, atol=1e-5) and torch.allclose(lse, lse_full, atol=1e-5)


def test_index_helpers_roundtrip():
    gen = torch.Generator().manual_seed(8)
    mask = torch.rand(2, 2, 5, 9, generator=gen) < 0.4
    index, nums = orc.mask_to_q2k(mask)
    bias_like = torch.zeros_like(mask)
    for b in range(2):
        for h in range(2):
            for m in range(5):
                bias_like[b, h, m, index[b, h, m, :int(nums[b, h, m])].long()] = True
    assert torch.equal(bias_like, mask)
    k2q, k2q_nums = orc.q2k_to_k2q(index, 0, 9, nums)
    for b in range(2):
        for h in range(2):
            for j in range(9):
                ids = torch.nonzero(mask[b, h, :, j]).flatten().int()
                assert int(k2q_nums[b, h, j]) == ids.numel()
                assert torch.equal(k2q[b, h, j, :ids.numel()], ids)
                assert (k2q[b, h, j, ids.numel():] == 0).all()
