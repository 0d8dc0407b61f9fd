"""CPU oracle for the block-sparse attention hot path (plain torch on CPU, fp32 unless stated).

TEST INFRASTRUCTURE.  Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm
may import this module; the product package never does.

Parity status: PINNED.  Every function below restates a function of the reference repository's own
test-suite / utilities (cited per function, paths relative to that repository) and is checked in
tests/test_oracle_golden.py against golden vectors produced by importing and running those very
functions (generator: tests/golden/make_golden.py), plus the reference tests' literal known-answer
cases (analytic softmax rows, CSR literal matrices, constant-V exact cases).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

NEG_INF = float("-inf")


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


# --------------------------------------------------------------------------------------------------
# dense-bias reference (small shapes)
# --------------------------------------------------------------------------------------------------
def block_sparse_to_attn_bias(q2k_block_index, block_sparse_num, block_sizes, seqlen_q, seqlen_k, blk_m=128,
                              blk_n=128, q2k_block_nums=None):
    """Additive bias [B,H,Sq,Sk]: 0 where (q block, kv block) is selected and the kv token is below the
    block's valid size, -inf elsewhere.  Restates tests/test_flash_fwd.py:138-186 (scatter of the first
    ``count`` index entries, block_sizes validity, clip to seqlen_k)."""
    B, H, Nq, _ = q2k_block_index.shape
    Nkv = block_sizes.shape[0]
    col = torch.arange(blk_n)
    block_valid = col.unsqueeze(0) < block_sizes.unsqueeze(1)  # [Nkv, blk_n]
    attended = torch.zeros(B, H, Nq, Nkv, dtype=torch.bool)
    if q2k_block_nums is None:
        attended.scatter_(3, q2k_block_index[..., :block_sparse_num].long(), True)
    else:
        for b in range(B):
            for h in range(H):
                for m in range(Nq):
                    n = int(q2k_block_nums[b, h, m])
                    attended[b, h, m].scatter_(0, q2k_block_index[b, h, m, :n].long(), True)
    token_valid = (attended.unsqueeze(-1) & block_valid).reshape(B, H, Nq, -1)[..., :seqlen_k]
    bias = torch.full((B, H, seqlen_q, seqlen_k), NEG_INF, dtype=torch.float32)
    for m in range(Nq):
        s, e = m * blk_m, min((m + 1) * blk_m, seqlen_q)
        if s >= seqlen_q:
            break
        bias[:, :, s:e] = torch.where(token_valid[:, :, m:m + 1], 0.0, NEG_INF)
    return bias


def unpack_gqa_attn_bias(bias_kv, nheads, group, seqlen_q):
    """Packed-GQA bias [B,Hkv,Sq*G(padded),Sk] -> per-query-head bias [B,Hq,Sq,Sk]; packed row r is
    (seq = r // G, head offset = r % G).  Restates tests/test_flash_fwd.py:189-215."""
    B, Hkv, rows, Sk = bias_kv.shape
    r = torch.arange(rows)
    seq, off = r // group, r % group
    out = torch.full((B, nheads, seqlen_q, Sk), NEG_INF, dtype=bias_kv.dtype)
    valid = seq < seqlen_q
    for g in range(group):
        sel = (off == g) & valid
        for hk in range(Hkv):
            out[:, hk * group + g, seq[sel]] = bias_kv[:, hk, r[sel]]
    return out


def attention_dense(q, k, v, attn_bias, softmax_scale=None, upcast=True, reorder_ops=False):
    """Dense masked attention on BHSD tensors; returns (out [B,Hq,Sq,D], lse [B,Hq,Sq] fp32).

    out restates utils/testing.py:323-434 (``attention_ref`` with ``attn_bias``: fp32 upcast, kv heads
    repeated for GQA, scale applied to q - or to k when ``reorder_ops`` -, softmax, P @ V, cast back);
    lse restates tests/test_flash_fwd.py:313-317 (logsumexp of the scaled, biased scores) and fully
    masked rows are zeroed as in :319-320."""
    dtype_og = q.dtype
    if upcast:
        q, k, v = q.float(), k.float(), v.float()
    G = q.shape[1] // k.shape[1]
    if G > 1:
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    if not reorder_ops:
        scores = torch.einsum("bhtd,bhsd->bhts", q * scale, k)
    else:
        scores = torch.einsum("bhtd,bhsd->bhts", q, k * scale)
    scores = scores + attn_bias.to(scores.dtype)
    attn = torch.softmax(scores, dim=-1).to(v.dtype)
    out = torch.einsum("bhts,bhsd->bhtd", attn, v)
    out = torch.nan_to_num(out, nan=0.0)
    lse = torch.logsumexp(scores.float(), dim=-1)
    return out.to(dtype_og), lse


# --------------------------------------------------------------------------------------------------
# gathered reference (large shapes): exactly the selected, valid tokens
# --------------------------------------------------------------------------------------------------
def _extent(sizes, b, h, j):
    if sizes is None:
        return None
    if sizes.ndim == 1:
        return int(sizes[j])
    if sizes.ndim == 2:
        return int(sizes[b, j])
    return int(sizes[b, h, j])


def attention_gathered(q, k, v, index, count, nums=None, sizes=None, scale=None, blk=128, heads=None,
                       batches=None, return_lse=True, tiles=None):
    """FP32 attention over exactly the selected valid KV tokens of every query block (MHA or unpacked GQA).

    Restates tests/test_bsa_fp8_blk128.py:45-77 (``sparse_reference``: live prefix of the index row,
    tokens < Sk, optional rank-1/2/3 block extents, empty rows -> 0) and
    tests/test_flash_fwd.py:473-523 (``_reference_variable_case``, which also yields the LSE, -inf for
    empty rows).  ``heads`` / ``batches`` / ``tiles`` restrict the computation to a subset (big configs)."""
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    out = torch.zeros((B, Hq, Sq, D), dtype=torch.float32)
    lse = torch.full((B, Hq, Sq), NEG_INF, dtype=torch.float32)
    Nq = index.shape[2]
    off = torch.arange(blk)
    for b in (range(B) if batches is None else batches):
        for h in (range(Hq) if heads is None else heads):
            hk = h // G
            kf, vf = k[b, hk].float(), v[b, hk].float()
            for m in (range(Nq) if tiles is None else tiles):
                n = count if nums is None else int(nums[b, h, m])
                n = max(0, min(n, index.shape[-1]))
                s, e = m * blk, min((m + 1) * blk, Sq)
                if n == 0 or s >= Sq:
                    continue
                toks = []
                for i in range(n):
                    j = int(index[b, h, m, i])
                    t = j * blk + off
                    ok = t < Sk
                    ext = _extent(sizes, b, hk, j)
                    if ext is not None:
                        ok = ok & (off < ext)
                    toks.append(t[ok])
                toks = torch.cat(toks)
                if toks.numel() == 0:
                    continue
                sc = (q[b, h, s:e].float() @ kf[toks].T) * scale
                out[b, h, s:e] = torch.softmax(sc, dim=-1) @ vf[toks]
                lse[b, h, s:e] = torch.logsumexp(sc, dim=-1)
    return (out, lse) if return_lse else out


def attention_gathered_packed(q, k, v, index, count, nums=None, sizes=None, scale=None, blk=128, kv_heads=None,
                              tiles=None):
    """Packed-GQA variant: ``index``/``nums`` are per (batch, kv head, packed tile); packed row r of a kv
    head is (seq = r // G, query head = hkv*G + r % G) (csrc/utils/pack_gqa.py:10-35,
    tests/test_flash_fwd.py:189-215, :273-274)."""
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    out = torch.zeros((B, Hq, Sq, D), dtype=torch.float32)
    lse = torch.full((B, Hq, Sq), NEG_INF, dtype=torch.float32)
    Nt = index.shape[2]
    off = torch.arange(blk)
    for b in range(B):
        for hk in (range(Hkv) if kv_heads is None else kv_heads):
            kf, vf = k[b, hk].float(), v[b, hk].float()
            # packed query matrix [Sq*G, D]
            qp = q[b, hk * G:(hk + 1) * G].float().permute(1, 0, 2).reshape(Sq * G, D)
            for m in (range(Nt) if tiles is None else tiles):
                n = count if nums is None else int(nums[b, hk, m])
                n = max(0, min(n, index.shape[-1]))
                s, e = m * blk, min((m + 1) * blk, Sq * G)
                if n == 0 or s >= Sq * G:
                    continue
                toks = []
                for i in range(n):
                    j = int(index[b, hk, m, i])
                    t = j * blk + off
                    ok = t < Sk
                    ext = _extent(sizes, b, hk, j)
                    if ext is not None:
                        ok = ok & (off < ext)
                    toks.append(t[ok])
                toks = torch.cat(toks)
                if toks.numel() == 0:
                    continue
                sc = (qp[s:e] @ kf[toks].T) * scale
                o = torch.softmax(sc, dim=-1) @ vf[toks]
                l = torch.logsumexp(sc, dim=-1)
                rows = torch.arange(s, e)
                out[b, hk * G + rows % G, rows // G] = o
                lse[b, hk * G + rows % G, rows // G] = l
    return out, lse


# --------------------------------------------------------------------------------------------------
# top-k index producer
# --------------------------------------------------------------------------------------------------
def block_mean(x, blk):
    """fp32 mean of every ``blk`` consecutive tokens of a BHSD tensor (a short tail averages what exists)."""
    B, H, S, D = x.shape
    N = ceil_div(S, blk)
    xf = x.float()
    out = torch.empty((B, H, N, D), dtype=torch.float32)
    for n in range(N):
        out[:, :, n] = xf[:, :, n * blk:(n + 1) * blk].mean(dim=2)
    return out


def topk_q2k(scores, topk):
    """ids of the ``topk`` largest scores per row, ascending; ties go to the lower id.  Restates the recipe of
    tests/bench_cutedsl_performance.py:150-167 (``torch.topk(sorted=False)`` then ``sort``) with a defined
    tie rule: a stable descending sort keeps equal scores in id order."""
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices[..., :topk]
    return order.sort(dim=-1).values.to(torch.int32)


# --------------------------------------------------------------------------------------------------
# backward reference
# --------------------------------------------------------------------------------------------------
def backward_dense(q, k, v, dout, attn_bias, softmax_scale, upcast=True):
    """torch-autograd backward of dense masked attention on BHSD tensors; returns
    (out, lse, dq, dk, dv).  Restates tests/test_flash_bwd.py:80-108 (``_torch_ref_bwd``)."""
    dtype = torch.float32 if upcast else q.dtype
    q_r = q.detach().to(dtype).requires_grad_()
    k_r = k.detach().to(dtype).requires_grad_()
    v_r = v.detach().to(dtype).requires_grad_()
    if upcast:
        scores = torch.einsum("bhtd,bhsd->bhts", q_r * softmax_scale, k_r)
    else:
        scores = torch.einsum("bhtd,bhsd->bhts", q_r, k_r * softmax_scale)
    scores = scores + attn_bias.to(scores.dtype)
    attn = torch.softmax(scores, dim=-1)
    out = torch.einsum("bhts,bhsd->bhtd", attn, v_r)
    out = torch.nan_to_num(out, nan=0.0)
    lse = torch.logsumexp(scores, dim=-1)
    out.backward(dout.to(dtype))
    return out.detach().to(dout.dtype), lse.detach().float(), q_r.grad.detach(), k_r.grad.detach(), v_r.grad.detach()


def backward_gathered(q, k, v, dout, index, count, nums=None, scale=None, blk=128, heads=None, batches=None,
                      sizes=None, upcast=True):
    """Gathered-form backward for large shapes (MHA): per query block, autograd through the softmax over
    exactly the selected tokens; gradients scattered back.  Same math as ``backward_dense`` (the dense
    bias only removes the unselected tokens), so it is validated against it on small cases.  ``sizes``
    (rank 1/2/3) are the valid-token counts of the KV blocks, as in ``attention_gathered``.  ``upcast=False``
    keeps the tile arithmetic in the inputs' own dtype (the "PyTorch implementation in bf16" whose distance
    from the fp32 result sets the reference's tolerance, tests/test_flash_bwd.py:53-61)."""
    cdt = torch.float32 if upcast else q.dtype
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    dq = torch.zeros((B, H, Sq, D), dtype=torch.float32)
    dk = torch.zeros((B, H, Sk, D), dtype=torch.float32)
    dv = torch.zeros((B, H, Sk, D), dtype=torch.float32)
    off = torch.arange(blk)
    for b in (range(B) if batches is None else batches):
        for h in (range(H) if heads is None else heads):
            kf, vf = k[b, h].to(cdt), v[b, h].to(cdt)
            for m in range(index.shape[2]):
                n = count if nums is None else int(nums[b, h, m])
                n = max(0, min(n, index.shape[-1]))
                s, e = m * blk, min((m + 1) * blk, Sq)
                if n == 0 or s >= Sq:
                    continue
                parts = []
                for i in range(n):
                    j = int(index[b, h, m, i])
                    ext = blk if sizes is None else max(0, min(blk, _extent(sizes, b, h, j)))
                    parts.append(j * blk + off[:ext])
                toks = torch.cat(parts)
                toks = toks[toks < Sk]
                if toks.numel() == 0:
                    continue
                qt = q[b, h, s:e].to(cdt)
                kt, vt = kf[toks], vf[toks]
                do = dout[b, h, s:e].to(cdt)
                p = torch.softmax((qt @ kt.T) * scale, dim=-1)
                dp = do @ vt.T
                delta = (p * dp).sum(-1, keepdim=True)
                ds = p * (dp - delta)
                dq[b, h, s:e] = ((ds @ kt) * scale).float()
                dk[b, h].index_add_(0, toks, ((ds.T @ qt) * scale).float())
                dv[b, h].index_add_(0, toks, (p.T @ do).float())
    return dq, dk, dv


# --------------------------------------------------------------------------------------------------
# index construction
# --------------------------------------------------------------------------------------------------
def mask_to_q2k(mask: torch.Tensor, cap: Optional[int] = None):
    """Block mask [B,H,Nq,Nkv] -> (index [B,H,Nq,cap] ascending, zero padded; nums).  Inverse of the
    scatter at tests/test_flash_fwd.py:156-170; counts above ``cap`` are clamped."""
    B, H, Nq, Nkv = mask.shape
    cap = Nkv if cap is None else cap
    index = torch.zeros((B, H, Nq, cap), dtype=torch.int32)
    nums = torch.zeros((B, H, Nq), dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            for m in range(Nq):
                ids = torch.nonzero(mask[b, h, m] != 0).flatten()[:cap]
                index[b, h, m, :ids.numel()] = ids.int()
                nums[b, h, m] = ids.numel()
    return index, nums


def q2k_to_k2q(q2k, block_sparse_num, num_kv_blocks, q2k_block_nums=None):
    """Dense k2q with set semantics: [B,H,Nkv,Nq] ascending q ids padded with zeros, and counts.
    Restates utils/block_sparse_index.py:20-68 (scatter into a kv-major byte map, then linear pack;
    the index entries read are position < count, ids outside [0,Nkv) are skipped)."""
    B, H, Nq, cap = q2k.shape
    k2q = torch.zeros((B, H, num_kv_blocks, Nq), dtype=torch.int32)
    k2q_nums = torch.zeros((B, H, num_kv_blocks), dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            bitmap = torch.zeros((num_kv_blocks, Nq), dtype=torch.bool)
            for m in range(Nq):
                n = block_sparse_num if q2k_block_nums is None else int(q2k_block_nums[b, h, m])
                n = max(0, min(n, cap))
                for i in range(n):
                    j = int(q2k[b, h, m, i])
                    if 0 <= j < num_kv_blocks:
                        bitmap[j, m] = True
            for j in range(num_kv_blocks):
                ids = torch.nonzero(bitmap[j]).flatten()
                k2q[b, h, j, :ids.numel()] = ids.int()
                k2q_nums[b, h, j] = ids.numel()
    return k2q, k2q_nums


def bucketed_k2q_csr(q2k, block_sparse_num, num_kv_blocks, bucket_size_blocks, q2k_block_nums=None):
    """Bucketed k2q CSR: (offsets [B,H,G,Nkv+1] int32, rows dict (b,h,g,kv) -> ascending list of q ids).
    Restates tests/test_bucketed_k2q_csr.py:12-74 (``_reference_bucketed_k2q``): one edge per occurrence
    at position < clamp(count, 0, cap) whose id is in [0,Nkv); offsets run on across the groups of one
    (b,h)."""
    B, H, Nq, cap = q2k.shape
    G = ceil_div(Nq, bucket_size_blocks)
    offsets = torch.empty((B, H, G, num_kv_blocks + 1), dtype=torch.int32)
    rows: Dict[Tuple[int, int, int, int], List[int]] = {}
    for b in range(B):
        for h in range(H):
            base = 0
            for g in range(G):
                group_rows: List[List[int]] = [[] for _ in range(num_kv_blocks)]
                for m in range(g * bucket_size_blocks, min(Nq, (g + 1) * bucket_size_blocks)):
                    n = block_sparse_num if q2k_block_nums is None else int(q2k_block_nums[b, h, m])
                    n = min(max(0, n), cap)
                    for i in range(n):
                        j = int(q2k[b, h, m, i])
                        if 0 <= j < num_kv_blocks:
                            group_rows[j].append(m)
                running = base
                for j, r in enumerate(group_rows):
                    offsets[b, h, g, j] = running
                    rows[(b, h, g, j)] = r
                    running += len(r)
                offsets[b, h, g, num_kv_blocks] = running
                base = running
    return offsets, rows


# --------------------------------------------------------------------------------------------------
# Sage FP8 quantisation
# --------------------------------------------------------------------------------------------------
def sage_quantize(q, k, v):
    """Closed-form Sage quantisation recipe on BF16 BHSD inputs (D = 128); returns
    (q8, k8, v8 as float8_e4m3fn, q_scale [B,H,Sq], k_scale [B,H,ceil(Sk/16)], v_scale [H,128]).
    Restates tests/test_bsa_fp8_quant.py:34-49: per-token Q scale with BF16-rounded reciprocal and
    product; K mean-centred over the sequence, scale per 16 tokens over all channels (zero-padded tail
    rows are centred too); V scale per (head, channel) over batch and sequence, FP32 reciprocal."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    qs = q.float().abs().amax(dim=-1).clamp_min(1e-3) / 448.0
    q8 = (q * qs.bfloat16().reciprocal()[..., None]).to(torch.float8_e4m3fn)
    vs = v.float().abs().amax(dim=(0, 2)).clamp_min(1e-3) / 448.0
    v8 = (v.float() * vs.reciprocal()[None, :, None, :]).to(torch.float8_e4m3fn)
    mean = k.float().mean(dim=2, keepdim=True)
    padded = torch.nn.functional.pad(k.float(), (0, 0, 0, (-Sk) % 16))
    centred = (padded - mean).reshape(B, H, -1, 16, 128)
    ks = centred.abs().amax(dim=(-1, -2)).clamp_min(1e-3) / 448.0
    k8 = (centred / ks[..., None, None]).to(torch.float8_e4m3fn).reshape(B, H, -1, 128)[:, :, :Sk]
    return q8, k8, v8, qs, ks, vs


def sage_dequantize(q8, k8, v8, qs, ks, vs):
    """BF16 dequantised Q/K/V (K without its mean: softmax is invariant to it).
    Restates tests/test_bsa_fp8_blk128.py:80-90."""
    B, H, Sq, D = q8.shape
    Sk = k8.shape[2]
    return (
        (q8.float() * qs.reshape(B, H, Sq, 1)).bfloat16(),
        (k8.float() * ks.reshape(B, H, -1).repeat_interleave(16, dim=-1)[..., :Sk, None]).bfloat16(),
        (v8.float() * vs.reshape(1, H, 1, D)).bfloat16(),
    )


def fp8_accuracy(out, ref):
    """(mean relative error, max abs error) as asserted by tests/test_bsa_fp8_blk128.py:93-101."""
    err = (out.float() - ref.float()).abs()
    return (err.mean() / ref.abs().mean().clamp_min(1e-8)).item(), err.max().item()


# --------------------------------------------------------------------------------------------------
# split-KV combine
# --------------------------------------------------------------------------------------------------
def combine_partials(partial_o, partial_lse):
    """LSE-weighted merge: partial_o [S,...,D], partial_lse [S,...] -> (out fp32, lse).  Math of
    csrc/fwd/sm100_blk64/bsa_fwd_combine.py:253-566 (all -inf rows give 0 / -inf, :458-468)."""
    m = partial_lse.amax(dim=0)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(partial_lse - m_safe)
    s = w.sum(dim=0)
    lse = torch.where(s > 0, m_safe + torch.log(s), torch.full_like(s, NEG_INF))
    wn = torch.where(s > 0, w / s.clamp_min(1e-38), torch.zeros_like(w))
    out = (torch.nan_to_num(partial_o, nan=0.0) * wn.unsqueeze(-1)).sum(dim=0)
    return out, lse


# --------------------------------------------------------------------------------------------------
# split / scheduler policy tables (pure host logic)
# --------------------------------------------------------------------------------------------------
def blk64_kv_splits_from_count(kv_blocks: int, max_kv_splits: int = 16) -> int:
    """bsa_attn_interface.py:676-690."""
    if kv_blocks >= 900:
        s = 8
    elif kv_blocks >= 450:
        s = 4
    elif kv_blocks >= 256:
        s = 2
    else:
        s = 1
    return max(1, min(s, max_kv_splits, kv_blocks))


def blk64_auto_kv_splits(batch, heads, seqlen_q, kv_blocks, max_kv_splits: int = 16) -> int:
    """bsa_attn_interface.py:649-673: one split as soon as B*H*ceil(Sq/64) >= 512."""
    if kv_blocks <= 1:
        return 1
    if batch * heads * ceil_div(seqlen_q, 64) >= 512:
        return 1
    return blk64_kv_splits_from_count(kv_blocks, max_kv_splits)


def blk64_auto_fp8_kv_splits(kv_blocks: int, heads: int, seqlen_q: int, batch: int, num_sms: int) -> int:
    """bsa_attn_interface.py:693-718: no split when the 64-row query tiles fill the SMs; otherwise the largest
    power of two <= 16 whose (tile, split) items still fit the SMs, reduced until each split keeps >= 8 blocks
    and a two-way split >= 128 blocks in total."""
    tiles = batch * heads * ceil_div(seqlen_q, 64)
    if tiles >= num_sms:
        return 1
    best = 1
    for s in (2, 4, 8, 16):
        if s * tiles <= num_sms:
            best = s
    for s in (16, 8, 4, 2):
        if s <= best and kv_blocks >= 8 * s and (s != 2 or kv_blocks >= 128):
            return s
    return 1


# --------------------------------------------------------------------------------------------------
# FLOP / byte conventions and the synthetic BASELINE workloads
# --------------------------------------------------------------------------------------------------
def sparse_flops(pairs: int, blk: int, d: int = 128, backward: bool = False) -> float:
    """4*blk^2*D per active pair forward, 10*blk^2*D backward (tests/bench_cutedsl_performance.py:336-355)."""
    return (10.0 if backward else 4.0) * pairs * blk * blk * d


def make_uniform_index(B, H, Nq, Nkv, count, gen, diagonal=True):
    """Each row: the diagonal block (when ``diagonal``) plus distinct uniform others, sorted ascending."""
    idx = torch.empty((B, H, Nq, count), dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            for m in range(Nq):
                if diagonal:
                    d = min(m, Nkv - 1)
                    perm = torch.randperm(Nkv - 1, generator=gen)[:count - 1]
                    others = perm + (perm >= d).long()
                    row = torch.cat([torch.tensor([d]), others])
                else:
                    row = torch.randperm(Nkv, generator=gen)[:count]
                idx[b, h, m] = torch.sort(row).values.int()
    return idx


def config1(seed: int = 0):
    """BASELINE config 1: B=1,H=4,S=1024,D=128 fp32, 8x8 grid of 128-blocks, diagonal + 1 other block,
    ascending int32 index, N(0,1) inputs, scale 1/sqrt(128)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, 4, 1024, 128, generator=g)
    k = torch.randn(1, 4, 1024, 128, generator=g)
    v = torch.randn(1, 4, 1024, 128, generator=g)
    idx = make_uniform_index(1, 4, 8, 8, 2, g)
    return q, k, v, idx, 2
