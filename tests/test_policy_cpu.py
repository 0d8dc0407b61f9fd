"""CPU: split / scheduler policies of the host mirror against the reference's tables.

The FP8 table is the reference's own test table (tests/test_bsa_fp8_fwd.py:17-66, read as text); the grid
was produced by running its function (tests/golden/make_golden.py).  No GPU is touched."""
import inspect

import pytest
import torch

from helpers import load_golden

FP8_TABLE = [  # (heads, seqlen_q, kv_blocks, expected) at batch 1, 148 SMs
    (4, 64, 1, 1), (4, 64, 31, 1), (4, 64, 127, 8), (4, 64, 128, 16), (4, 64, 548, 16), (8, 64, 188, 16),
    (8, 64, 1089, 16), (1, 64 * 37, 32, 4), (1, 64 * 74, 127, 1), (1, 64 * 74, 128, 2), (1, 64 * 100, 2048, 1),
    (1, 64 * 148, 2048, 1), (4, 119040, 188, 1), (8, 349440, 548, 1), (4, 579840, 909, 1), (8, 695040, 1089, 1),
    (4, 49290 + 2216 + 752, 915, 1),
]


def _iface():
    from block_sparse_attention import bsa_attn_interface
    return bsa_attn_interface


@pytest.mark.parametrize("heads,seqlen_q,kv_blocks,expected", FP8_TABLE)
def test_fp8_auto_split_table(heads, seqlen_q, kv_blocks, expected):
    assert _iface()._sm100_blk64_auto_fp8_kv_splits(kv_blocks, heads, seqlen_q, 1, 148) == expected


def test_fp8_auto_split_batch_and_sm_count():
    f = _iface()._sm100_blk64_auto_fp8_kv_splits
    assert (f(188, 4, 64, 1, 148), f(188, 4, 64, 8, 148), f(188, 4, 64, 37, 148)) == (16, 4, 1)
    assert (f(2048, 1, 64 * 100, 1, 148), f(2048, 1, 64 * 100, 1, 200)) == (1, 2)


def test_fp8_auto_split_grid_from_reference():
    f = _iface()._sm100_blk64_auto_fp8_kv_splits
    for kv_blocks, heads, seqlen_q, batch, num_sms, splits in load_golden("policy_fp8_blk64_splits.npz")["rows"].tolist():
        assert f(kv_blocks, heads, seqlen_q, batch, num_sms) == splits


def test_bf16_split_table_from_reference():
    g = load_golden("policy_blk64_splits.npz")
    f = _iface()._sm100_blk64_kv_splits_from_count
    for c, s in zip(g["counts"].tolist(), g["splits"].tolist()):
        assert f(c) == s


def test_split_offsets_cover_every_row():
    """Boundaries of the in-kernel split rule: start at 0, end at the count, never decrease, and every inner
    boundary is even (a KV iteration consumes two 64-token blocks)."""
    f = _iface()._build_sm100_blk64_kv_split_offsets
    nums = torch.tensor([[[0, 1, 2, 7, 8, 33, 256]]], dtype=torch.int32)
    for splits in (1, 2, 3, 4, 16):
        off = f(nums, 0, 1, 1, 7, splits, torch.device("cpu"))
        assert off.shape == (1, 1, 7, splits + 1) and off.dtype == torch.int32
        assert (off[..., 0] == 0).all() and (off[..., -1] == nums).all()
        assert (off[..., 1:] >= off[..., :-1]).all()
        assert (off[..., 1:-1] % 2 == 0).all()
    uniform = f(None, 10, 2, 3, 4, 2, torch.device("cpu"))
    assert uniform.shape == (2, 3, 4, 3) and uniform[0, 0, 0].tolist() == [0, 4, 10]
    with pytest.raises(AssertionError):
        f(nums, 0, 1, 1, 7, 0, torch.device("cpu"))


def test_workspace_policy_passes_through_without_a_device():
    f = _iface()._resolve_blk64_split_workspace
    q = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16)
    assert f(q, 128, 1, False) == 1 and f(q, 128, 8, True) == 8  # CPU tensor: nothing to measure
    assert _iface()._blk64_split_workspace_bytes(q, 128, 4) == 4 * 256 * 129 * 4 + 256 * (128 * 2 + 4)


def test_use_clc_chooser_keeps_the_reference_signature():
    f = _iface().choose_blk64_use_clc
    assert list(inspect.signature(f).parameters) == ["q", "block_sparse_num", "q2k_block_nums", "layout"]
    q = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16)
    assert f(q, 8) is False and f(q, 300, torch.ones(1, 2, 2, dtype=torch.int32), layout="bshd") is False
    with pytest.raises(AssertionError):
        f(q, 8, layout="sbhd")
