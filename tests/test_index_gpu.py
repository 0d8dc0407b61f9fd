"""GPU parity (bit-exact) of the index kernels against the CPU oracle and the reference's CSR model."""
import numpy as np
import pytest
import torch

from helpers import load_golden
from oracle import bsa_oracle as orc

pytestmark = pytest.mark.gpu


def _assert_csr(q2k, bsn, nkv, bucket, nums):
    from block_sparse_attention.bsa_attn_interface import _build_bucketed_k2q_csr
    offsets, indices, G, rows_per_group = _build_bucketed_k2q_csr(
        q2k.cuda(), bsn, nkv, bucket_size_blocks=bucket, q2k_block_nums=None if nums is None else nums.cuda())
    exp_off, exp_rows = orc.bucketed_k2q_csr(q2k, bsn, nkv, bucket, nums)
    assert offsets.dtype == torch.int32 and indices.dtype == torch.int32
    assert G == exp_off.shape[2] and rows_per_group == nkv
    width = q2k.shape[3] if nums is not None else bsn  # the reference's shapes (bsa_attn_interface.py:3999-4019)
    assert indices.shape[-1] == max(1, q2k.shape[2] * width)
    assert torch.equal(offsets.cpu(), exp_off)
    off, idx = offsets.cpu(), indices.cpu()
    B, H = off.shape[:2]
    for b in range(B):
        for h in range(H):
            for g in range(G):
                for j in range(nkv):
                    row = idx[b, h, off[b, h, g, j]:off[b, h, g, j + 1]].tolist()
                    assert row == sorted(exp_rows[(b, h, g, j)]), (b, h, g, j)  # already ascending
    return offsets, indices


@pytest.mark.parametrize("name", ["csr_literal_variable.npz", "csr_random_fixed.npz", "csr_topk_1025.npz"])
def test_csr_golden(name):
    g = load_golden(name)
    q2k = torch.from_numpy(g["q2k"])
    nums = torch.from_numpy(g["nums"]) if g["nums"].size else None
    offsets, _ = _assert_csr(q2k, int(g["bsn"]), int(g["nkv"]), int(g["bucket"]), nums)
    assert np.array_equal(offsets.cpu().numpy(), g["offsets"])


def test_csr_empty_edge_width():
    """tests/test_bucketed_k2q_csr.py:225-243: zero-width index."""
    q2k = torch.empty((1, 1, 2, 0), dtype=torch.int32)
    nums = torch.zeros((1, 1, 2), dtype=torch.int32)
    _assert_csr(q2k, 0, 3, 1, nums)


def test_csr_config2_shape_deterministic():
    gen = torch.Generator().manual_seed(0)
    q2k = orc.make_uniform_index(1, 2, 256, 256, 26, gen)
    o1, i1 = _assert_csr(q2k, 26, 256, 384, None)
    o2, i2 = _assert_csr(q2k, 26, 256, 100, None)  # three query groups
    from block_sparse_attention.bsa_attn_interface import _build_bucketed_k2q_csr
    o3, i3, _, _ = _build_bucketed_k2q_csr(q2k.cuda(), 26, 256, bucket_size_blocks=384)
    assert torch.equal(o1, o3) and torch.equal(i1[..., :256 * 26], i3[..., :256 * 26])
    with pytest.raises(AssertionError):
        _build_bucketed_k2q_csr(q2k.cuda(), 27, 256, bucket_size_blocks=384)  # count above the row width


def test_csr_long_rows_global_sort_path():
    """every q block selects kv block 0: one CSR row of 1500 entries (> the shared-memory sort limit)."""
    q2k = torch.zeros((1, 1, 1500, 2), dtype=torch.int32)
    q2k[..., 1] = 1
    _assert_csr(q2k, 2, 3, 2000, None)


def test_csr_attention_sink_rows_at_the_default_bucket():
    """One KV block (an attention sink) is selected by every query block: with the default 64-token bucket of
    1152 query blocks its CSR row has 1152 entries in the first group and the rest in the second.  Rows of
    that length are sorted by counting in shared memory; the build must stay in the tens of microseconds."""
    from block_sparse_attention.bsa_attn_interface import _build_bucketed_k2q_csr
    gen = torch.Generator().manual_seed(9)
    Nq, Nkv = 1300, 40
    others = torch.stack([torch.randperm(Nkv - 1, generator=gen)[:3] + 1 for _ in range(2 * Nq)]).reshape(1, 2, Nq, 3)
    q2k = torch.cat([others[..., :1], torch.zeros(1, 2, Nq, 1, dtype=torch.long), others[..., 1:]], dim=-1).int()
    _assert_csr(q2k, 4, Nkv, 1152, None)
    dup = q2k.clone()
    dup[0, 0, 5, 2] = 0  # a duplicated id stays a duplicate
    _assert_csr(dup, 4, Nkv, 1152, None)
    qc = q2k.cuda()
    _build_bucketed_k2q_csr(qc, 4, Nkv, bucket_size_blocks=1152)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(10):
        _build_bucketed_k2q_csr(qc, 4, Nkv, bucket_size_blocks=1152)
    b.record()
    torch.cuda.synchronize()
    assert a.elapsed_time(b) / 10 < 1.0, "CSR build with 1152-entry rows took more than 1 ms"


def test_q2k_to_k2q_set_semantics():
    from block_sparse_attention import convert_q2k_to_k2q
    gen = torch.Generator().manual_seed(2)
    q2k = torch.randint(-1, 14, (2, 3, 9, 7), generator=gen, dtype=torch.int32)  # duplicates, -1 and 13 out of range
    nums = torch.randint(-1, 9, (2, 3, 9), generator=gen, dtype=torch.int32)
    for n in (None, nums):
        k2q, k2q_nums = convert_q2k_to_k2q(q2k.cuda(), 5, 13, None if n is None else n.cuda())
        e_k2q, e_nums = orc.q2k_to_k2q(q2k, 5, 13, n)
        assert torch.equal(k2q.cpu(), e_k2q) and torch.equal(k2q_nums.cpu(), e_nums)


def test_mask_to_q2k_roundtrip_and_clamp():
    from block_sparse_attention import block_mask_to_q2k
    gen = torch.Generator().manual_seed(4)
    mask = torch.rand(2, 2, 37, 300, generator=gen) < 0.1
    mask[0, 0, 0] = False
    mask[1, 1, 5] = True
    index, nums = block_mask_to_q2k(mask.cuda())
    e_index, e_nums = orc.mask_to_q2k(mask)
    assert torch.equal(index.cpu(), e_index) and torch.equal(nums.cpu(), e_nums)
    index, nums = block_mask_to_q2k(mask.cuda(), max_kv_blocks=16)
    e_index, e_nums = orc.mask_to_q2k(mask, 16)
    assert torch.equal(index.cpu(), e_index) and torch.equal(nums.cpu(), e_nums)


@pytest.mark.parametrize("rows,cap", [(5, 3), (1024, 8), (5000, 256), (40000, 57)])
def test_lpt_order_is_the_stable_descending_sort(rows, cap):
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    gen = torch.Generator().manual_seed(rows)
    nums = torch.randint(-2, cap + 3, (rows,), generator=gen, dtype=torch.int32)
    order = torch.empty(rows, dtype=torch.int32, device="cuda")
    scratch = torch.empty(int(lib.bsa_lpt_order_scratch_ints(rows, cap)), dtype=torch.int32, device="cuda")
    nc = nums.cuda()
    rc = lib.bsa_lpt_order(nc.data_ptr(), rows, cap, order.data_ptr(), scratch.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    expected = torch.sort(nums.clamp(0, cap), descending=True, stable=True).indices.int()
    assert torch.equal(order.cpu(), expected)
