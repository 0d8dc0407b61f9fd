"""Host API of the B200-native block-sparse attention engine.

Function names, argument order, defaults, return conventions and error types mirror the reference's
``bsa_attn_interface.py`` (``bsa_attn_fwd`` :3428, ``bsa_attn_bwd`` :3759, ``bsa_fp8_blk128_fwd`` :3352,
``bsa_fp8_fwd`` :3386, ``bsa_fp8_blk64_fwd`` :2953, ``convert_q2k_to_k2q`` :3726,
``_build_bucketed_k2q_csr`` :3999) so that callers and tests written against the reference run unchanged.
Below the signatures nothing is shared with it: there is no JIT, no AOT loader and no kernel cache -
each call validates, allocates outputs/workspaces as torch tensors and makes one or two calls into
``libbsa_b200.so`` on the current CUDA stream.  Argument validation raises ``AssertionError`` like the
reference; a missing library or a workspace that cannot be allocated raises ``RuntimeError``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _cabi

__all__ = [
    "bsa_attn_fwd",
    "bsa_attn_bwd",
    "bsa_fp8_fwd",
    "bsa_fp8_blk64_fwd",
    "bsa_fp8_blk128_fwd",
    "convert_q2k_to_k2q",
    "block_mask_to_q2k",
    "choose_blk64_use_clc",
    "check_device_status",
]


def maybe_contiguous(x):
    """Same rule as the reference (bsa_attn_interface.py:145-146): only the last stride has to be 1."""
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _ceil_div(a: int, b: int) -> int:
    return (int(a) + int(b) - 1) // int(b)


def _tma_ready(t: torch.Tensor, elt: int) -> torch.Tensor:
    """Returns a BHSD view the tensor maps can address: 16-byte aligned base, non-zero strides that are
    multiples of 16 bytes, unit last stride.  Copies only when the given view cannot be addressed."""
    unit = 16 // elt
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0
    for d in range(3):
        s = t.stride(d)
        if t.shape[d] > 1 and (s <= 0 or s % unit != 0):
            ok = False
    if not ok:
        return t.contiguous()
    if any(t.shape[d] == 1 and (t.stride(d) <= 0 or t.stride(d) % unit != 0) for d in range(3)):
        # a size-1 dimension may carry any stride; give it a valid one without copying
        strides = list(t.stride())
        for d in (2, 1, 0):
            if t.shape[d] == 1:
                strides[d] = strides[d + 1] * t.shape[d + 1] if d < 2 else t.shape[3]
                if strides[d] % unit != 0 or strides[d] <= 0:
                    return t.contiguous()
        return t.as_strided(t.shape, strides)
    return t


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Synchronises and raises RuntimeError if a kernel reported an expired bounded wait."""
    _cabi.check_status(device)


# --------------------------------------------------------------------------------------------------
# split / scheduler policies (reference: bsa_attn_interface.py:649-690, :2061-2092)
# --------------------------------------------------------------------------------------------------
def _sm100_blk64_kv_splits_from_count(kv_blocks: int, max_kv_splits: int = 16) -> int:
    kv_blocks = int(kv_blocks)
    if kv_blocks >= 900:
        splits = 8
    elif kv_blocks >= 450:
        splits = 4
    elif kv_blocks >= 256:
        splits = 2
    else:
        splits = 1
    return max(1, min(int(splits), int(max_kv_splits), kv_blocks))


def _sm100_blk64_auto_kv_splits(q: torch.Tensor, q2k_block_index: torch.Tensor, fixed_block_sparse_num: int,
                                max_kv_splits: int = 16) -> int:
    """``kv_splits="auto"``: one split when the query tiles alone fill the GPU (>= 512 tiles), otherwise
    2/4/8 splits at >= 256/450/900 blocks per row."""
    if not q.is_cuda:
        return 1
    kv_blocks = int(fixed_block_sparse_num)
    if kv_blocks <= 0:
        kv_blocks = int(q2k_block_index.shape[-1])
    if kv_blocks <= 1:
        return 1
    batch, heads, seqlen_q, _ = q.shape
    if batch * heads * _ceil_div(seqlen_q, 64) >= 512:
        return 1
    return _sm100_blk64_kv_splits_from_count(kv_blocks, max_kv_splits)


def _sm100_blk64_auto_fp8_kv_splits(kv_blocks: int, heads: int, seqlen_q: int, batch: int, num_sms: int) -> int:
    """Automatic split count of the Sage FP8 64-token forward (reference bsa_attn_interface.py:693-718,
    table in its tests/test_bsa_fp8_fwd.py:17-66).  The kernel runs one persistent CTA per SM, so splitting
    the KV range only pays when the query tiles alone leave SMs idle: the count doubles while twice as
    many (tile, split) items still fit the SMs, up to 16, and is halved again until every split keeps at
    least 8 blocks (two splits: at least 128 blocks in total).  ``kv_blocks`` is the largest per-tile
    block count."""
    kv_blocks, num_sms = int(kv_blocks), int(num_sms)
    tiles = int(batch) * int(heads) * _ceil_div(int(seqlen_q), 64)
    if tiles >= num_sms:
        return 1
    splits = 1
    while splits < 16 and 2 * splits * tiles <= num_sms:
        splits *= 2
    while splits > 1:
        enough = kv_blocks >= 8 * splits and not (splits == 2 and kv_blocks < 128)
        if enough:
            break
        splits //= 2
    return splits


def _build_sm100_blk64_kv_split_offsets(q2k_block_nums: Optional[torch.Tensor], uniform_block_sparse_num: int,
                                        batch_size: int, num_heads: int, num_q_blocks: int, kv_splits: int,
                                        device: torch.device) -> torch.Tensor:
    """Split boundaries ``[B, H, Nq, kv_splits + 1]`` (int32, in 64-token blocks) of the 64-token forward.

    The reference builds this tensor on the host and hands it to its kernel (bsa_attn_interface.py:779-823,
    8-block-aligned because its kernel consumes eight blocks per step).  Here the kernel derives the
    boundaries itself from the row count - split ``s`` takes KV iterations ``[n*s/k, n*(s+1)/k)`` of the
    row's ``n = ceil(count / 2)`` two-block iterations - so no tensor is needed on the hot path; this
    function returns exactly those boundaries for callers and tests that want to see them."""
    assert 1 <= kv_splits <= 256, "kv_splits must be in [1, 256]"
    if q2k_block_nums is not None and q2k_block_nums.numel() > 0:
        counts = q2k_block_nums.to(device=device, dtype=torch.int64).clamp_min(0)
    else:
        counts = torch.full((batch_size, num_heads, num_q_blocks), int(uniform_block_sparse_num),
                            dtype=torch.int64, device=device)
    iters = (counts + 1) // 2
    s = torch.arange(kv_splits + 1, dtype=torch.int64, device=device)
    bounds = 2 * ((iters[..., None] * s) // kv_splits)
    return torch.minimum(bounds, counts[..., None]).to(torch.int32).contiguous()


def _blk64_split_workspace_bytes(q: torch.Tensor, value_dim: int, kv_splits: int) -> int:
    """Bytes a split run keeps alive: FP32 partial O and LSE of every split plus the final output and LSE."""
    batch, heads, seqlen_q, _ = q.shape
    rows = batch * heads * seqlen_q
    return int(kv_splits * rows * (value_dim + 1) * 4 + rows * (value_dim * q.element_size() + 4))


def _resolve_blk64_split_workspace(q: torch.Tensor, value_dim: int, kv_splits: int, allow_fallback: bool) -> int:
    """Fits the split count to the memory that can still be allocated (reference bsa_attn_interface.py:841-873):
    free device memory plus what the caching allocator holds unused, minus a reserve of 5 % of the device
    (at least 512 MiB).  An automatic count is halved until it fits; an explicit one raises RuntimeError."""
    kv_splits = int(kv_splits)
    if kv_splits <= 1 or not q.is_cuda:
        return kv_splits
    free_bytes, total_bytes = torch.cuda.mem_get_info(q.device)
    cached = max(0, torch.cuda.memory_reserved(q.device) - torch.cuda.memory_allocated(q.device))
    budget = max(0, free_bytes + cached - max(512 << 20, int(0.05 * total_bytes)))
    fit = kv_splits
    while fit > 1:
        need = _blk64_split_workspace_bytes(q, value_dim, fit)
        if need <= budget:
            return fit
        if not allow_fallback:
            raise RuntimeError(
                f"blk64 split-KV kv_splits={kv_splits} requires about {need / (1 << 30):.2f} GiB of live "
                f"workspace, but only {budget / (1 << 30):.2f} GiB is available after the safety reserve; "
                "lower kv_splits")
        fit //= 2
    return 1


def choose_blk64_use_clc(q: torch.Tensor, block_sparse_num: int, q2k_block_nums: Optional[torch.Tensor] = None,
                         layout: str = "bhsd") -> bool:
    """Same signature as the reference's scheduler chooser (bsa_attn_interface.py:2061-2066), which picks
    between its static and its hardware work-stealing (CLC) launch.  This engine has one scheduler - a
    persistent grid walking a longest-first work list - so there is nothing to choose and the answer is
    always False; ``use_clc`` is accepted by ``bsa_attn_fwd`` and has no effect."""
    assert layout in ("bhsd", "bshd"), f"layout must be 'bhsd' or 'bshd', got {layout!r}"
    assert q.dim() == 4
    return False


def sm100_blk128_bwd_default_bucketed_k2q_size_blocks(num_q_blocks: int, num_heads: int) -> int:
    """Default query-group size of the backward CSR (csrc/bwd/sm100_blk128/bsa_bwd_sm100.py:2162-2171)."""
    if num_q_blocks >= 4096 and num_heads <= 1:
        return 256
    if num_q_blocks >= 2048:
        return 512
    return 384


def sm100_bwd_default_bucketed_k2q_size_blocks(num_q_blocks: int) -> int:
    """Default query-group size of the 64-token backward CSR (csrc/bwd/sm100_blk64/bsa_bwd_sm100.py:21-24)."""
    if num_q_blocks < 2048 or num_q_blocks >= 8192:
        return 1088
    return 1152


# --------------------------------------------------------------------------------------------------
# shared forward launcher
# --------------------------------------------------------------------------------------------------
def _normalise_metadata(q2k_block_index, block_sizes, q2k_block_nums, device):
    assert q2k_block_index.dtype == torch.int32, "q2k_block_index must be int32"
    assert q2k_block_index.ndim == 4, "q2k_block_index must be (batch, heads, q_blocks, max_kv_blocks)"
    assert q2k_block_index.device == device
    q2k_block_index = q2k_block_index.contiguous()
    has_sizes = block_sizes is not None and block_sizes.numel() > 0
    if has_sizes:
        assert block_sizes.dtype == torch.int32, "block_sizes must be int32"
        assert block_sizes.device == device
        block_sizes = block_sizes.contiguous()
    else:
        block_sizes = None
    has_nums = q2k_block_nums is not None and q2k_block_nums.numel() > 0
    if has_nums:
        assert q2k_block_nums.dtype == torch.int32, "q2k_block_nums must be int32"
        assert q2k_block_nums.ndim == 3, (
            f"q2k_block_nums must be 3D (batch, num_heads, num_q_blocks), got {q2k_block_nums.ndim}D")
        assert q2k_block_nums.device == device
        q2k_block_nums = q2k_block_nums.contiguous()
    else:
        q2k_block_nums = None
    return q2k_block_index, block_sizes, q2k_block_nums


def _block_size_strides(block_sizes, batch, heads, num_kv_blocks, allow_ranks):
    if block_sizes is None:
        return 0, 0
    assert block_sizes.ndim in allow_ranks, f"block_sizes rank {block_sizes.ndim} not supported here"
    if block_sizes.ndim == 1:
        assert block_sizes.shape == (num_kv_blocks,), (
            f"block_sizes must have {num_kv_blocks} entries, got {tuple(block_sizes.shape)}")
        return 0, 0
    if block_sizes.ndim == 2:
        assert block_sizes.shape == (batch, num_kv_blocks)
        return num_kv_blocks, 0
    assert block_sizes.shape == (batch, heads, num_kv_blocks)
    return heads * num_kv_blocks, num_kv_blocks


def _lpt_order(lib, counts: torch.Tensor, cap: int) -> torch.Tensor:
    """Longest-first order of the rows of an int32 count tensor (stable; counts clamped to [0, cap])."""
    device = counts.device
    rows = counts.numel()
    cap_sort = max(1, min(int(cap), 32000))
    order = torch.empty(rows, dtype=torch.int32, device=device)
    scratch = torch.empty(max(1, int(lib.bsa_lpt_order_scratch_ints(rows, cap_sort))), dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _cabi.check(lib.bsa_lpt_order(counts.data_ptr(), rows, cap_sort, order.data_ptr(), scratch.data_ptr(),
                                      _cabi.stream_ptr(device)), "bsa_lpt_order")
    return order


def _launch_fwd(*, q, k, v, out, lse, q2k_block_index, q2k_block_nums, block_sizes, bs_strides, blk,
                block_sparse_num, pack_gqa, splits, softmax_scale, dtype_code, q_scale=None, k_scale=None,
                v_scale=None):
    """q, k, v, out are BHSD views.  Runs the producer and, for splits > 1, the combine."""
    lib = _cabi.load()
    device = q.device
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    elt = 1 if dtype_code == _cabi.BSA_DTYPE_E4M3 else 2
    q_k, k_k, v_k = _tma_ready(q, elt), _tma_ready(k, elt), _tma_ready(v, elt)
    out_k = out if (out.stride(-1) == 1 and out.data_ptr() % 16 == 0 and
                    all(out.shape[d] == 1 or (out.stride(d) > 0 and out.stride(d) % 8 == 0) for d in range(3))) \
        else None
    out_tmp = out_k if out_k is not None else torch.empty(out.shape, dtype=out.dtype, device=device)
    out_tmp_view = _tma_ready(out_tmp, 2)
    lse_k = lse
    if lse is not None and not lse.is_contiguous():
        lse_k = torch.empty(lse.shape, dtype=torch.float32, device=device)

    args = _cabi.FwdArgs()
    args.q, args.k, args.v = q_k.data_ptr(), k_k.data_ptr(), v_k.data_ptr()
    args.out = out_tmp_view.data_ptr()
    args.lse = _cabi.ptr(lse_k)
    args.q2k_index = q2k_block_index.data_ptr()
    args.q2k_nums = _cabi.ptr(q2k_block_nums)
    args.block_sizes = _cabi.ptr(block_sizes)
    args.q_scale, args.k_scale, args.v_scale = _cabi.ptr(q_scale), _cabi.ptr(k_scale), _cabi.ptr(v_scale)
    args.status = _cabi.status_buffer(device).data_ptr()
    args.q_stride = _cabi.strides3(q_k)
    args.k_stride = _cabi.strides3(k_k)
    args.v_stride = _cabi.strides3(v_k)
    args.o_stride = _cabi.strides3(out_tmp_view)
    args.bs_stride_b, args.bs_stride_h = bs_strides
    args.dtype = dtype_code
    args.blk = blk
    args.B, args.Hq, args.Hkv, args.Sq, args.Sk, args.D = B, Hq, Hkv, Sq, Sk, D
    args.cap = q2k_block_index.shape[-1]
    args.block_sparse_num = int(block_sparse_num)
    args.pack_gqa = 1 if pack_gqa else 0
    args.splits = int(splits)
    args.softmax_scale = float(softmax_scale)
    work_order = None
    if q2k_block_nums is not None and q2k_block_nums.numel() > 2 * lib.bsa_num_sms(device.index or 0):
        # variable counts: longest-first work order so that the persistent CTAs finish together
        work_order = _lpt_order(lib, q2k_block_nums, int(args.cap))
        args.work_order = work_order.data_ptr()
    partial_o = partial_lse = None
    if splits > 1:
        try:
            partial_o = torch.empty((splits, B, Hq, Sq, D), dtype=torch.float32, device=device)
            partial_lse = torch.empty((splits, B, Hq, Sq), dtype=torch.float32, device=device)
        except torch.OutOfMemoryError as e:  # same error class as the reference's workspace check (:868-873)
            raise RuntimeError(f"split-KV workspace for kv_splits={splits} does not fit: {e}") from e
        args.partial_o, args.partial_lse = partial_o.data_ptr(), partial_lse.data_ptr()
    stream = _cabi.stream_ptr(device)
    with torch.cuda.device(device):
        torch.cuda.nvtx.range_push("bsa_attn_fwd_kernel")
        try:
            _cabi.check(lib.bsa_fwd(args, stream), "bsa_fwd")
            if splits > 1:
                import ctypes
                ostr = (ctypes.c_int64 * 3)(out_tmp_view.stride(0), out_tmp_view.stride(1), out_tmp_view.stride(2))
                _cabi.check(lib.bsa_fwd_combine(partial_o.data_ptr(), partial_lse.data_ptr(),
                                                out_tmp_view.data_ptr(), _cabi.ptr(lse_k), splits, B, Hq, Sq, D,
                                                ostr, stream), "bsa_fwd_combine")
        finally:
            torch.cuda.nvtx.range_pop()
    if out_tmp is not out:
        out.copy_(out_tmp)
    if lse is not None and lse_k is not lse:
        lse.copy_(lse_k)
    return out, lse


# --------------------------------------------------------------------------------------------------
# BF16 forward
# --------------------------------------------------------------------------------------------------
def bsa_attn_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    q2k_block_index: torch.Tensor,
    block_sparse_num: int,
    block_sizes: Optional[torch.Tensor] = None,
    q2k_block_nums: Optional[torch.Tensor] = None,
    allow_empty_block_nums: bool = True,
    softmax_scale: Optional[float] = None,
    pack_gqa: Optional[bool] = None,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    layout: str = "bhsd",
    *,
    sparse_block_size: int = 64,
    use_clc: Optional[bool] = None,
    kv_splits: int | str = 1,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Block-sparse attention forward; always returns ``(out, lse_or_None)``.

    Same contract as the reference (bsa_attn_interface.py:3428-3720 for 128-token blocks, :2330-2841 for
    64-token blocks): only the first ``count`` entries of each ``q2k_block_index`` row are read
    (``count`` = ``q2k_block_nums[b,h,m]`` or ``block_sparse_num``), ``block_sizes`` masks the tail tokens
    of KV blocks, rows with no live block give ``out = 0`` and ``lse = -inf``, LSE is the natural log of
    the scaled scores' partition sum and is returned iff ``return_lse``, a gradient is required or an
    ``lse`` buffer was passed.  ``block_sizes`` may have rank 1 ``(Nkv,)``, 2 ``(B, Nkv)`` or 3 ``(B, Hkv, Nkv)``
    for both block sizes.  BF16 (FP16 with 128-token blocks); D = 128, or 64 / 96 with 128-token blocks
    (those ride on the 128-wide tiles: the tensor maps zero-fill the missing channels).  Relaxations over the reference: odd fixed counts are
    accepted for 128-token blocks and the physical KV tail is always masked.
    """
    assert sparse_block_size in (64, 128), f"sparse_block_size must be 64 or 128, got {sparse_block_size}"
    assert layout in ("bhsd", "bshd"), f"layout must be 'bhsd' or 'bshd', got {layout!r}"
    requires_grad = q.requires_grad or k.requires_grad or v.requires_grad
    return_lse_result = return_lse or requires_grad or lse is not None
    blk = sparse_block_size
    if blk == 64:
        assert pack_gqa is None, "pack_gqa is only supported for sparse_block_size=128"
        auto = isinstance(kv_splits, str)
        if auto:
            assert kv_splits == "auto", "kv_splits string value must be 'auto'"
        else:
            assert int(kv_splits) >= 1, "kv_splits must be >= 1"
    else:
        assert use_clc is None, "use_clc is only supported for sparse_block_size=64"
        assert kv_splits == 1, "kv_splits is only supported for sparse_block_size=64"
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4
    assert q.is_cuda and k.is_cuda and v.is_cuda, "inputs must be on CUDA device"
    assert q.device == k.device == v.device, "Q/K/V must be on the same CUDA device"
    assert q.dtype == k.dtype == v.dtype, "inputs must have the same dtype"
    assert q.dtype in (torch.float16, torch.bfloat16), "inputs must be float16 or bfloat16"
    if q.dtype == torch.float16:
        assert sparse_block_size == 128, "sparse_block_size=64 requires Q/K/V to all use bf16"
    q, k, v = [maybe_contiguous(t) for t in (q, k, v)]
    qb, kb, vb = (q, k, v) if layout == "bhsd" else (q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    B, Hq, Sq, D = qb.shape
    Bk, Hkv, Sk, Dk = kb.shape
    assert vb.shape == kb.shape and Bk == B and Dk == D
    if blk == 128:
        # same set as the reference's 128-token forward (csrc/fwd/sm100_blk128/bsa_fwd_sm100.py:75-78)
        assert D in (64, 96, 128), f"head dimension must be 64, 96 or 128 for sparse_block_size=128, got {D}"
    else:
        assert D == 128, "sparse_block_size=64 requires head dimension 128"
    assert Hq % Hkv == 0
    G = Hq // Hkv
    if blk == 64:
        assert Hq == Hkv, "sparse_block_size=64 supports MHA only"
    device = q.device
    q2k_block_index, block_sizes, q2k_block_nums = _normalise_metadata(
        q2k_block_index, block_sizes, q2k_block_nums, device)

    packed = (G > 1 and blk % G == 0) if pack_gqa is None else bool(pack_gqa)
    if blk == 64 or G == 1:
        packed = False
    if packed:
        assert blk % G == 0, "pack_gqa needs the block size to be a multiple of the group size"
    Hidx = Hkv if packed else Hq
    Nq = _ceil_div(Sq * G, blk) if packed else _ceil_div(Sq, blk)
    Nkv = _ceil_div(Sk, blk)
    assert q2k_block_index.shape[:3] == (B, Hidx, Nq), (
        f"q2k_block_index has shape {tuple(q2k_block_index.shape)}, expected ({B}, {Hidx}, {Nq}, max_kv_blocks)")
    if q2k_block_nums is not None:
        assert q2k_block_nums.shape == (B, Hidx, Nq)
        if not allow_empty_block_nums and not torch.cuda.is_current_stream_capturing():
            assert int(q2k_block_nums.min()) >= 1, "q2k_block_nums must be >= 1 when allow_empty_block_nums=False"
    else:
        assert block_sparse_num >= 1, f"block_sparse_num={block_sparse_num} must be >= 1"
        assert q2k_block_index.shape[-1] >= block_sparse_num, (
            f"q2k_block_index last dim ({q2k_block_index.shape[-1]}) must be >= block_sparse_num ({block_sparse_num})")
    bs_strides = _block_size_strides(block_sizes, B, Hkv, Nkv, (1, 2, 3))
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)

    out_shape = (B, Hq, Sq, D) if layout == "bhsd" else (B, Sq, Hq, D)
    if out is None:
        out = torch.empty(out_shape, dtype=q.dtype, device=device)
    else:
        assert out.shape == out_shape
        assert out.dtype == q.dtype and out.device == device
        assert out.stride(-1) == 1
    lse_shape = (B, Hq, Sq)
    if lse is None:
        lse_buf = torch.empty(lse_shape, dtype=torch.float32, device=device) if return_lse_result else None
    else:
        assert lse.shape == lse_shape
        assert lse.dtype == torch.float32 and lse.device == device
        lse_buf = lse
    out_b = out if layout == "bhsd" else out.transpose(1, 2)

    splits = 1
    if blk == 64:
        if isinstance(kv_splits, str):
            splits = _sm100_blk64_auto_kv_splits(qb, q2k_block_index,
                                                 0 if q2k_block_nums is not None else block_sparse_num)
        else:
            splits = int(kv_splits)
        splits = max(1, min(splits, 256))
        splits = _resolve_blk64_split_workspace(qb, D, splits, allow_fallback=isinstance(kv_splits, str))

    _launch_fwd(q=qb, k=kb, v=vb, out=out_b, lse=lse_buf, q2k_block_index=q2k_block_index,
                q2k_block_nums=q2k_block_nums, block_sizes=block_sizes, bs_strides=bs_strides, blk=blk,
                block_sparse_num=block_sparse_num if q2k_block_nums is None else 0, pack_gqa=packed,
                splits=splits, softmax_scale=softmax_scale,
                dtype_code=_cabi.BSA_DTYPE_F16 if q.dtype == torch.float16 else _cabi.BSA_DTYPE_BF16)
    return out, (lse_buf if return_lse_result else None)


# --------------------------------------------------------------------------------------------------
# Sage FP8 forward
# --------------------------------------------------------------------------------------------------
def _bsa_fp8_blk128_fwd(q_fp8, k_fp8, v_fp8, q_sfs, k_sfs, v_sfs, q2k_block_index, topk_num, softmax_scale,
                        block_sizes, q2k_block_nums, kv_splits, blk=128):
    assert isinstance(kv_splits, int) and not isinstance(kv_splits, bool), "kv_splits must be an int"
    assert 1 <= kv_splits <= 256, "kv_splits must be in [1, 256]"
    for t in (q_fp8, k_fp8, v_fp8):
        assert t.dtype == torch.float8_e4m3fn, "Q/K/V must be float8_e4m3fn"
        assert t.is_cuda and t.dim() == 4
    q8, k8, v8 = q_fp8.contiguous(), k_fp8.contiguous(), v_fp8.contiguous()
    B, H, Sq, D = q8.shape
    assert B >= 1 and H >= 1, "Sage FP8 requires positive batch and head counts"
    assert D == 128, "Sage FP8 requires D=128"
    assert k8.shape[:2] == (B, H) and k8.shape[3] == D and v8.shape == k8.shape, "MHA with matching K/V shapes"
    Sk = k8.shape[2]
    device = q8.device
    for s in (q_sfs, k_sfs, v_sfs):
        assert s.dtype == torch.float32 and s.device == device
    assert q_sfs.numel() == B * H * Sq, f"q scale must hold B*H*Sq = {B * H * Sq} values"
    assert k_sfs.numel() == B * H * _ceil_div(Sk, 16), "k scale must hold B*H*ceil(Sk/16) values"
    assert v_sfs.numel() == H * D, "v scale must hold H*D values"
    q_sc = q_sfs.reshape(B, H, Sq).contiguous()
    k_sc = k_sfs.reshape(B, H, _ceil_div(Sk, 16)).contiguous()
    v_sc = v_sfs.reshape(H, D).contiguous()
    q2k_block_index, block_sizes, q2k_block_nums = _normalise_metadata(
        q2k_block_index, block_sizes, q2k_block_nums, device)
    Nq, Nkv = _ceil_div(Sq, blk), _ceil_div(Sk, blk)
    assert q2k_block_index.shape[:3] == (B, H, Nq)
    if q2k_block_nums is not None:
        assert q2k_block_nums.shape == (B, H, Nq)
    else:
        assert topk_num >= 1 and q2k_block_index.shape[-1] >= topk_num
    bs_strides = _block_size_strides(block_sizes, B, H, Nkv, (1, 2, 3))
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    out = torch.empty((B, H, Sq, D), dtype=torch.bfloat16, device=device)
    _launch_fwd(q=q8, k=k8, v=v8, out=out, lse=None, q2k_block_index=q2k_block_index,
                q2k_block_nums=q2k_block_nums, block_sizes=block_sizes, bs_strides=bs_strides, blk=blk,
                block_sparse_num=topk_num if q2k_block_nums is None else 0, pack_gqa=False, splits=kv_splits,
                softmax_scale=softmax_scale, dtype_code=_cabi.BSA_DTYPE_E4M3, q_scale=q_sc, k_scale=k_sc,
                v_scale=v_sc)
    return out


def bsa_fp8_blk128_fwd(
    q_fp8: torch.Tensor,
    k_fp8: torch.Tensor,
    v_fp8: torch.Tensor,
    q_sfs: torch.Tensor,
    k_sfs: torch.Tensor,
    v_sfs: torch.Tensor,
    q2k_block_index: torch.Tensor,
    topk_num: int,
    softmax_scale: Optional[float] = None,
    *,
    block_sizes: Optional[torch.Tensor] = None,
    q2k_block_nums: Optional[torch.Tensor] = None,
    kv_splits: int = 1,
) -> torch.Tensor:
    """Sage FP8 forward with 128-token blocks; returns one BF16 BHSD tensor
    (reference bsa_attn_interface.py:3352-3383).  Scales are the multiplicative dequantisation factors of
    ``quantize_sage_bhsd``: Q per token, K per 16 tokens, V per (head, channel); they may arrive flattened."""
    return _bsa_fp8_blk128_fwd(q_fp8, k_fp8, v_fp8, q_sfs, k_sfs, v_sfs, q2k_block_index, topk_num,
                               softmax_scale, block_sizes, q2k_block_nums, kv_splits)


def bsa_fp8_blk64_fwd(
    q_fp8: torch.Tensor,
    k_fp8: torch.Tensor,
    v_fp8: torch.Tensor,
    q_sfs: torch.Tensor,
    k_sfs: torch.Tensor,
    v_sfs: torch.Tensor,
    q2k_block_index: torch.Tensor,
    topk_num: int,
    softmax_scale: Optional[float] = None,
    *,
    block_sizes: Optional[torch.Tensor] = None,
    q2k_block_nums: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Sage FP8 forward with 64-token blocks (reference bsa_attn_interface.py:2953-3182): same scale
    recipe and metadata as the 128-block entry; returns one BF16 BHSD tensor.  The split count is chosen
    here by the reference's automatic FP8 policy (``_sm100_blk64_auto_fp8_kv_splits``) from the row width of
    the index, so a short-Q call that cannot fill the SMs with query tiles is split over the KV range; no
    device value is read back."""
    assert q_fp8.is_cuda and q_fp8.dim() == 4
    B, H, Sq, _ = q_fp8.shape
    has_nums = q2k_block_nums is not None and q2k_block_nums.numel() > 0
    width = int(q2k_block_index.shape[-1]) if has_nums else int(topk_num)
    num_sms = int(_cabi.load().bsa_num_sms(q_fp8.device.index or 0))
    splits = _sm100_blk64_auto_fp8_kv_splits(width, H, Sq, B, num_sms)
    splits = _resolve_blk64_split_workspace(q_fp8, 128, splits, allow_fallback=True)
    return _bsa_fp8_blk128_fwd(q_fp8, k_fp8, v_fp8, q_sfs, k_sfs, v_sfs, q2k_block_index, topk_num,
                               softmax_scale, block_sizes, q2k_block_nums, splits, blk=64)


def bsa_fp8_fwd(
    q_fp8: torch.Tensor,
    k_fp8: torch.Tensor,
    v_fp8: torch.Tensor,
    q_sfs: torch.Tensor,
    k_sfs: torch.Tensor,
    v_sfs: torch.Tensor,
    q2k_block_index: torch.Tensor,
    topk_num: int,
    softmax_scale: Optional[float] = None,
    *,
    sparse_block_size: int = 64,
    block_sizes: Optional[torch.Tensor] = None,
    q2k_block_nums: Optional[torch.Tensor] = None,
    kv_splits: int = 1,
) -> torch.Tensor:
    """Sage FP8 forward with explicit block size (reference bsa_attn_interface.py:3386-3425)."""
    assert sparse_block_size in (64, 128), "sparse_block_size must be 64 or 128"
    if sparse_block_size == 64:
        assert kv_splits == 1, "Explicit kv_splits is supported for blk128 only"
        return bsa_fp8_blk64_fwd(q_fp8, k_fp8, v_fp8, q_sfs, k_sfs, v_sfs, q2k_block_index, topk_num,
                                 softmax_scale, block_sizes=block_sizes, q2k_block_nums=q2k_block_nums)
    return _bsa_fp8_blk128_fwd(q_fp8, k_fp8, v_fp8, q_sfs, k_sfs, v_sfs, q2k_block_index, topk_num,
                               softmax_scale, block_sizes, q2k_block_nums, kv_splits)


# --------------------------------------------------------------------------------------------------
# index construction
# --------------------------------------------------------------------------------------------------
def block_mask_to_q2k(block_mask: torch.Tensor, max_kv_blocks: Optional[int] = None
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Boolean / uint8 block mask ``[B, H, Nq, Nkv]`` -> ``(q2k_block_index [B,H,Nq,cap] int32 ascending,
    q2k_block_nums [B,H,Nq] int32)``.  The reference has no such function; this is the inverse of the
    scatter its tests use to rebuild a mask from the index (tests/test_flash_fwd.py:156-170)."""
    assert block_mask.is_cuda and block_mask.ndim == 4
    assert block_mask.dtype in (torch.bool, torch.uint8)
    lib = _cabi.load()
    m = block_mask.contiguous().view(torch.uint8) if block_mask.dtype == torch.bool else block_mask.contiguous()
    B, H, Nq, Nkv = m.shape
    cap = Nkv if max_kv_blocks is None else int(max_kv_blocks)
    assert cap >= 1
    index = torch.empty((B, H, Nq, cap), dtype=torch.int32, device=m.device)
    nums = torch.empty((B, H, Nq), dtype=torch.int32, device=m.device)
    with torch.cuda.device(m.device):
        _cabi.check(lib.bsa_mask_to_q2k(m.data_ptr(), index.data_ptr(), nums.data_ptr(), B, H, Nq, Nkv, cap,
                                        _cabi.stream_ptr(m.device)), "bsa_mask_to_q2k")
    return index, nums


def convert_q2k_to_k2q(
    q2k_block_index: torch.Tensor,
    block_sparse_num: int,
    num_kv_blocks: int,
    q2k_block_nums: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverts the q2k index into the dense k2q layout (reference bsa_attn_interface.py:3726-3756):
    ``k2q_block_index [B,H,Nkv,Nq]`` ascending q ids padded with zeros, ``k2q_block_nums [B,H,Nkv]``."""
    assert q2k_block_index.is_cuda and q2k_block_index.dtype == torch.int32 and q2k_block_index.ndim == 4
    lib = _cabi.load()
    q2k = q2k_block_index.contiguous()
    B, H, Nq, cap = q2k.shape
    nums = None
    if q2k_block_nums is not None and q2k_block_nums.numel() > 0:
        assert q2k_block_nums.dtype == torch.int32 and q2k_block_nums.shape == (B, H, Nq)
        nums = q2k_block_nums.contiguous()
    k2q = torch.empty((B, H, num_kv_blocks, Nq), dtype=torch.int32, device=q2k.device)
    k2q_nums = torch.empty((B, H, num_kv_blocks), dtype=torch.int32, device=q2k.device)
    with torch.cuda.device(q2k.device):
        _cabi.check(lib.bsa_q2k_to_k2q(q2k.data_ptr(), _cabi.ptr(nums), int(block_sparse_num), B, H, Nq, cap,
                                       int(num_kv_blocks), k2q.data_ptr(), k2q_nums.data_ptr(),
                                       _cabi.stream_ptr(q2k.device)), "bsa_q2k_to_k2q")
    return k2q, k2q_nums


def _build_bucketed_k2q_csr(
    q2k_block_index: torch.Tensor,
    block_sparse_num: int,
    num_kv_blocks: int,
    *,
    bucket_size_blocks: int = 1152,
    q2k_block_nums: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, int, int]:
    """Bucketed k2q CSR (reference bsa_attn_interface.py:3999-4019): returns
    ``(offsets [B,H,G,Nkv+1], indices [B,H,max(1,Nq*W)], num_q_groups, num_kv_blocks)`` with ``W`` the fixed
    ``block_sparse_num`` or, with per-row counts, the row width of the index - the reference's shapes.  Unlike
    the reference every CSR row comes out in ascending q order, so the result is run-to-run identical."""
    offsets, indices, G = _build_k2q_csr_full(q2k_block_index, block_sparse_num, num_kv_blocks, bucket_size_blocks,
                                              q2k_block_nums)
    has_nums = q2k_block_nums is not None and q2k_block_nums.numel() > 0
    if not has_nums:
        Nq, cap = q2k_block_index.shape[2], q2k_block_index.shape[3]
        assert 0 <= block_sparse_num <= cap, (
            f"block_sparse_num ({block_sparse_num}) must not exceed the index row width ({cap})")
        indices = indices[..., :max(1, Nq * int(block_sparse_num))]
    return offsets, indices, G, int(num_kv_blocks)


def _build_k2q_csr_full(q2k_block_index, block_sparse_num, num_kv_blocks, bucket_size_blocks, q2k_block_nums):
    """The CSR with ``indices`` at its full allocation ``[B,H,max(1,Nq*cap)]`` (what ``bsa_bwd`` addresses)."""
    assert q2k_block_index.is_cuda and q2k_block_index.dtype == torch.int32 and q2k_block_index.ndim == 4
    assert bucket_size_blocks >= 1
    lib = _cabi.load()
    q2k = q2k_block_index.contiguous()
    B, H, Nq, cap = q2k.shape
    nums = None
    if q2k_block_nums is not None and q2k_block_nums.numel() > 0:
        assert q2k_block_nums.dtype == torch.int32 and q2k_block_nums.shape == (B, H, Nq)
        nums = q2k_block_nums.contiguous()
    G = _ceil_div(Nq, bucket_size_blocks)
    offsets = torch.empty((B, H, G, num_kv_blocks + 1), dtype=torch.int32, device=q2k.device)
    indices = torch.empty((B, H, max(1, Nq * cap)), dtype=torch.int32, device=q2k.device)
    with torch.cuda.device(q2k.device):
        _cabi.check(lib.bsa_build_k2q_csr(_cabi.ptr(q2k) if cap > 0 else None, _cabi.ptr(nums),
                                          int(block_sparse_num), B, H, Nq, cap, int(num_kv_blocks),
                                          int(bucket_size_blocks), offsets.data_ptr(), indices.data_ptr(),
                                          _cabi.stream_ptr(q2k.device)), "bsa_build_k2q_csr")
    return offsets, indices, G


# --------------------------------------------------------------------------------------------------
# backward
# --------------------------------------------------------------------------------------------------
_last_bwd_workspace = {}  # profiling only: the workspace of the last call made with a `stages` mask, per device


def bsa_attn_bwd(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    q2k_block_index: torch.Tensor,
    block_sparse_num: int,
    block_sizes: Optional[torch.Tensor] = None,
    q2k_block_nums: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    dq: Optional[torch.Tensor] = None,
    dk: Optional[torch.Tensor] = None,
    dv: Optional[torch.Tensor] = None,
    bucket_size_blocks: Optional[int] = None,
    layout: str = "bhsd",
    *,
    sparse_block_size: int = 64,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward of ``bsa_attn_fwd``; see ``_bsa_attn_bwd`` (same arguments plus a profiling knob)."""
    return _bsa_attn_bwd(dout, q, k, v, out, lse, q2k_block_index, block_sparse_num, block_sizes, q2k_block_nums,
                         softmax_scale, dq, dk, dv, bucket_size_blocks, layout, sparse_block_size=sparse_block_size)


def _bsa_attn_bwd(dout, q, k, v, out, lse, q2k_block_index, block_sparse_num, block_sizes=None, q2k_block_nums=None,
                  softmax_scale=None, dq=None, dk=None, dv=None, bucket_size_blocks=None, layout="bhsd", *,
                  sparse_block_size=64, stages=0):
    """Backward of ``bsa_attn_fwd`` (reference bsa_attn_interface.py:3759-3996; the 64-token driver is
    ``_bsa_attn_bwd_bucketed_k2q_csr`` :4022-4290): BF16, MHA, D = 128, 64- or 128-token blocks.  dQ, dK
    and dV are accumulated in tensor memory in a fixed order without atomics, so repeated calls are
    bit-identical.  ``block_sizes`` (rank 1 ``(num_kv_blocks,)`` or rank 2 ``(batch, num_kv_blocks)``)
    masks the tail tokens of KV blocks exactly as the forward does; the physical KV tail is always masked.
    The reference's 128-token backward ignores ``block_sizes``; with the full-block sizes its tests pass
    the results are the same.  ``stages`` (0 = everything) is a mask of the three passes to launch - 1 preprocess,
    2 dQ, 4 dK/dV - so that one pass can be timed alone after a full call has filled the workspace statistics."""
    assert sparse_block_size in (64, 128), f"sparse_block_size must be 64 or 128, got {sparse_block_size}"
    assert layout in ("bhsd", "bshd"), f"layout must be 'bhsd' or 'bshd', got {layout!r}"
    blk = sparse_block_size
    q, k, v, out, dout = [maybe_contiguous(t) for t in (q, k, v, out, dout)]
    if block_sizes is not None and block_sizes.numel() == 0:
        block_sizes = None
    if q2k_block_nums is not None and q2k_block_nums.numel() == 0:
        q2k_block_nums = None
    assert q.dtype == torch.bfloat16, "bwd only supports bfloat16"
    assert q.dtype == k.dtype == v.dtype == out.dtype == dout.dtype
    assert lse.dtype == torch.float32
    assert all(t.is_cuda for t in (q, k, v, out, dout, lse))
    tr = (lambda t: t) if layout == "bhsd" else (lambda t: None if t is None else t.transpose(1, 2))
    qb, kb, vb, ob, dob = tr(q), tr(k), tr(v), tr(out), tr(dout)
    B, H, Sq, D = qb.shape
    Bk, Hk, Sk, Dk = kb.shape
    assert Hk == H, "bwd does not support GQA/MQA"
    assert Bk == B and vb.shape == kb.shape and Dk == D
    if D == 64:
        # the reference's rule (bsa_attn_interface.py:3867-3873): a 64-wide head needs the 128-token path
        assert blk == 128, ("head_dim=64 bwd only supports the 128-token path; pass q2k_block_index sized to "
                            "sparse_block_size=128")
    else:
        assert D == 128, f"bwd only supports head_dim in {{64, 128}}, got {D}"
    assert ob.shape == qb.shape and dob.shape == qb.shape
    assert lse.shape == (B, H, Sq)
    device = q.device
    Nq, Nkv = _ceil_div(Sq, blk), _ceil_div(Sk, blk)
    if block_sizes is not None:
        assert block_sizes.dtype == torch.int32 and block_sizes.device == device
        block_sizes = block_sizes.contiguous()
    bs_strides = _block_size_strides(block_sizes, B, H, Nkv, (1, 2, 3))
    assert q2k_block_index.dtype == torch.int32
    assert q2k_block_index.shape[:3] == (B, H, Nq), (
        f"q2k_block_index has shape {tuple(q2k_block_index.shape)}, expected (b={B}, h={H}, num_q_blocks={Nq}, "
        "max_kv_blocks)")
    if q2k_block_nums is not None:
        assert q2k_block_nums.dtype == torch.int32
        assert q2k_block_nums.shape == (B, H, Nq)
        q2k_block_nums = q2k_block_nums.contiguous()
    else:
        assert q2k_block_index.shape[-1] >= block_sparse_num, (
            f"q2k_block_index last dim ({q2k_block_index.shape[-1]}) must be >= block_sparse_num "
            f"({block_sparse_num})")
    q2k_block_index = q2k_block_index.contiguous()
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    if bucket_size_blocks is None or bucket_size_blocks <= 0:
        bucket_size_blocks = (sm100_blk128_bwd_default_bucketed_k2q_size_blocks(Nq, H) if blk == 128
                              else sm100_bwd_default_bucketed_k2q_size_blocks(Nq))

    def _grad(buf, like):
        shape = like.shape
        if buf is None:
            return torch.empty(shape, dtype=like.dtype, device=device), None
        assert buf.shape == shape and buf.dtype == like.dtype and buf.is_cuda
        return buf, buf

    dq_t, _ = _grad(dq, q)
    dk_t, _ = _grad(dk, k)
    dv_t, _ = _grad(dv, v)
    dqb, dkb, dvb = tr(dq_t), tr(dk_t), tr(dv_t)

    lib = _cabi.load()
    offsets, indices, G = _build_k2q_csr_full(q2k_block_index, block_sparse_num, Nkv, bucket_size_blocks,
                                              q2k_block_nums)
    ws_bytes = int(lib.bsa_bwd_workspace_bytes(B, H, Sq, Sk, D))
    if stages not in (0, 7) and _last_bwd_workspace.get(device) is not None \
            and _last_bwd_workspace[device].numel() == max(ws_bytes, 16):
        workspace = _last_bwd_workspace[device]  # the row statistics of the full call before
    else:
        workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    if stages != 0:
        _last_bwd_workspace[device] = workspace

    views = {}
    for name, t in (("dout", dob), ("q", qb), ("k", kb), ("v", vb), ("out", ob)):
        views[name] = _tma_ready(t, 2)
    outs = {}
    copies = []
    for name, t in (("dq", dqb), ("dk", dkb), ("dv", dvb)):
        r = _tma_ready(t, 2)
        if r.data_ptr() != t.data_ptr() or r.stride() != t.stride():
            copies.append((t, r))
        outs[name] = r
    lse_c = lse.contiguous()

    a = _cabi.BwdArgs()
    a.dout, a.q, a.k, a.v, a.out = (views[n].data_ptr() for n in ("dout", "q", "k", "v", "out"))
    a.lse = lse_c.data_ptr()
    a.dq, a.dk, a.dv = outs["dq"].data_ptr(), outs["dk"].data_ptr(), outs["dv"].data_ptr()
    a.q2k_index = q2k_block_index.data_ptr()
    a.q2k_nums = _cabi.ptr(q2k_block_nums)
    a.csr_offsets, a.csr_indices = offsets.data_ptr(), indices.data_ptr()
    a.block_sizes = _cabi.ptr(block_sizes)
    a.bs_stride_b, a.bs_stride_h = bs_strides
    order_q = order_kv = None
    if q2k_block_nums is not None and q2k_block_nums.numel() > 2 * lib.bsa_num_sms(device.index or 0):
        # variable counts: both kernels walk their work items longest first, so the persistent CTAs finish
        # together (query tiles by their count, KV blocks by the number of query tiles that attend them)
        order_q = _lpt_order(lib, q2k_block_nums, q2k_block_index.shape[-1])
        per_block = (offsets[..., 1:] - offsets[..., :-1]).sum(dim=2, dtype=torch.int32).contiguous()
        order_kv = _lpt_order(lib, per_block, Nq)
    a.work_order_q, a.work_order_kv = _cabi.ptr(order_q), _cabi.ptr(order_kv)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.status = _cabi.status_buffer(device).data_ptr()
    a.do_stride, a.q_stride = _cabi.strides3(views["dout"]), _cabi.strides3(views["q"])
    a.k_stride, a.v_stride = _cabi.strides3(views["k"]), _cabi.strides3(views["v"])
    a.o_stride = _cabi.strides3(views["out"])
    a.dq_stride, a.dk_stride, a.dv_stride = (_cabi.strides3(outs[n]) for n in ("dq", "dk", "dv"))
    a.blk = blk
    a.B, a.H, a.Sq, a.Sk, a.D = B, H, Sq, Sk, D
    a.cap = q2k_block_index.shape[-1]
    a.block_sparse_num = int(block_sparse_num) if q2k_block_nums is None else 0
    a.num_q_groups = G
    a.bucket_size_blocks = int(bucket_size_blocks)
    a.softmax_scale = float(softmax_scale)
    a.stages = int(stages)
    with torch.cuda.device(device):
        torch.cuda.nvtx.range_push("bsa_attn_bwd_bucketed_k2q_csr_kernel")
        try:
            _cabi.check(lib.bsa_bwd(a, _cabi.stream_ptr(device)), "bsa_bwd")
        finally:
            torch.cuda.nvtx.range_pop()
    for dst, src in copies:
        dst.copy_(src)
    return dq_t, dk_t, dv_t
