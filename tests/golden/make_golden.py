"""Generates the golden vectors under tests/golden/ by importing and running the REFERENCE repository's
own CPU-runnable functions (its dense ``attention_ref``, the bias builders and gathered references of
its tests, its CSR model, its Sage dequantiser, its autograd backward reference and its split policy).

Run once where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/Block-Sparse-Attention

The outputs are small ``.npz`` files committed next to this script; tests/test_oracle_golden.py checks
the CPU oracle against them and the GPU tests check the CUDA path against the oracle.  Inputs are
BF16-representable and stored as raw 16-bit patterns; nothing here is copied from the reference's
sources - only the results of calling it.
"""
from __future__ import annotations

import argparse
import hashlib
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy()


def rand_bf16(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    sys.path.insert(0, os.path.join(ref, "tests"))
    sys.path.insert(0, ref)
    repo = os.path.dirname(os.path.dirname(HERE))
    sys.path.append(repo)  # for oracle.* generators only (appended: the reference package wins)

    from utils.testing import attention_ref  # noqa: E402
    import test_flash_fwd as tff  # noqa: E402
    import test_flash_bwd as tfb  # noqa: E402
    import test_bucketed_k2q_csr as tcsr  # noqa: E402
    import test_bsa_fp8_blk128 as tf8  # noqa: E402
    import test_bsa_fp8_fwd as tf8b  # noqa: E402
    import bsa_attn_interface as ref_iface  # noqa: E402
    from oracle import bsa_oracle as orc  # noqa: E402

    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---------------------------------------------------------------- A. dense forward, variable counts + block sizes
    g = torch.Generator().manual_seed(1234)
    for blk in (128, 64):
        B, H, Sq, Sk = 2, 2, 320, 448
        Nq, Nkv = math.ceil(Sq / blk), math.ceil(Sk / blk)
        q, k, v = rand_bf16(g, B, H, Sq, 128), rand_bf16(g, B, H, Sk, 128), rand_bf16(g, B, H, Sk, 128)
        nums = torch.randint(0, Nkv + 1, (B, H, Nq), generator=g, dtype=torch.int32)
        nums[0, 0, 0] = 0
        nums[1, 1, -1] = Nkv
        index = torch.zeros((B, H, Nq, Nkv), dtype=torch.int32)
        for b in range(B):
            for h in range(H):
                for m in range(Nq):
                    index[b, h, m] = torch.randperm(Nkv, generator=g).int()
        sizes = torch.randint(1, blk + 1, (Nkv,), generator=g, dtype=torch.int32)
        sizes[-1] = min(int(sizes[-1]), Sk - (Nkv - 1) * blk)
        bias = tff.block_sparse_to_attn_bias(index, 0, sizes, Sq, Sk, blk_m=blk, blk_n=blk, q2k_block_nums=nums)
        qb, kb, vb = (t.transpose(1, 2) for t in (q, k, v))  # the reference helper takes B,S,H,D
        out, _ = attention_ref(qb, kb, vb, None, None, attn_bias=bias, causal=False)
        scale = 1.0 / math.sqrt(128)
        scores = torch.einsum("bthd,bshd->bhts", qb.float() * scale, kb.float()) + bias
        lse = torch.logsumexp(scores, dim=-1)
        out = torch.nan_to_num(out.float(), nan=0.0).transpose(1, 2).contiguous()
        np.savez_compressed(os.path.join(HERE, f"fwd_dense_blk{blk}.npz"), q=bf16_bits(q), k=bf16_bits(k),
                            v=bf16_bits(v), index=index.numpy(), nums=nums.numpy(), sizes=sizes.numpy(),
                            bias_finite=torch.isfinite(bias).numpy().astype(np.uint8) if blk == 128 else np.zeros(1, np.uint8),
                            out=out.numpy(), lse=lse.numpy())

    # ---------------------------------------------------------------- B. BASELINE config 1 through the reference
    q, k, v, idx, n = orc.config1(seed=0)
    sizes = torch.full((8,), 128, dtype=torch.int32)
    bias = tff.block_sparse_to_attn_bias(idx, n, sizes, 1024, 1024, 128, 128)
    qb, kb, vb = (t.transpose(1, 2) for t in (q, k, v))
    out, _ = attention_ref(qb, kb, vb, None, None, attn_bias=bias, causal=False)
    scores = torch.einsum("bthd,bshd->bhts", qb.float() / math.sqrt(128), kb.float()) + bias
    lse = torch.logsumexp(scores, dim=-1)
    out = out.transpose(1, 2).contiguous()
    sha = hashlib.sha256(q.numpy().tobytes() + k.numpy().tobytes() + v.numpy().tobytes()
                         + idx.numpy().tobytes()).hexdigest()
    np.savez_compressed(os.path.join(HERE, "fwd_config1.npz"), input_sha256=np.array(sha), index=idx.numpy(),
                        out_rows=out[:, :, ::8].numpy(), lse=lse.numpy())

    # ---------------------------------------------------------------- C. packed GQA bias
    g = torch.Generator().manual_seed(77)
    B, Hq, Hkv, Sq, Sk = 1, 4, 2, 192, 256
    G = Hq // Hkv
    Nt, Nkv = math.ceil(Sq * G / 128), 2
    q, k, v = rand_bf16(g, B, Hq, Sq, 128), rand_bf16(g, B, Hkv, Sk, 128), rand_bf16(g, B, Hkv, Sk, 128)
    nums = torch.tensor([[[1, 2, 0], [2, 1, 2]]], dtype=torch.int32)
    index = torch.tensor([[[[1, 0], [0, 1], [1, 1]], [[1, 0], [0, 0], [0, 1]]]], dtype=torch.int32)
    sizes = torch.tensor([128, 100], dtype=torch.int32)
    bias_kv = tff.block_sparse_to_attn_bias(index, 0, sizes, Nt * 128, Sk, 128, 128, q2k_block_nums=nums)
    bias = tff.pack_gqa_attn_bias(bias_kv, Hq, G, Sq)
    qb, kb, vb = (t.transpose(1, 2) for t in (q, k, v))
    out, _ = attention_ref(qb, kb, vb, None, None, attn_bias=bias, causal=False)
    kexp = kb.float().repeat_interleave(G, dim=2)
    scores = torch.einsum("bthd,bshd->bhts", qb.float() / math.sqrt(128), kexp) + bias
    lse = torch.logsumexp(scores, dim=-1)
    out = torch.nan_to_num(out.float(), nan=0.0).transpose(1, 2).contiguous()
    np.savez_compressed(os.path.join(HERE, "fwd_packed_gqa.npz"), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                        index=index.numpy(), nums=nums.numpy(), sizes=sizes.numpy(), out=out.numpy(),
                        lse=lse.numpy())

    # ---------------------------------------------------------------- D. gathered variable-count reference
    g = torch.Generator().manual_seed(5)
    Sq, Sk, blk = 256, 512, 64
    q, k, v = rand_bf16(g, 1, 1, Sq, 128), rand_bf16(g, 1, 1, Sk, 128), rand_bf16(g, 1, 1, Sk, 128)
    nums = torch.tensor([[[0, 1, 3, 8]]], dtype=torch.int32)
    index = torch.stack([torch.randperm(8, generator=g) for _ in range(4)]).int().reshape(1, 1, 4, 8)
    sizes = torch.tensor([64, 1, 17, 63, 64, 32, 64, 5], dtype=torch.int32)
    out, lse = tff._reference_variable_case(q, k, v, index, nums, sizes, blk)
    np.savez_compressed(os.path.join(HERE, "fwd_gathered_blk64.npz"), q=bf16_bits(q), k=bf16_bits(k),
                        v=bf16_bits(v), index=index.numpy(), nums=nums.numpy(), sizes=sizes.numpy(),
                        out=out.numpy(), lse=lse.numpy())

    # ---------------------------------------------------------------- E. bucketed CSR model
    def csr_case(name, q2k, bsn, nkv, bucket, nums):
        offsets, rows = tcsr._reference_bucketed_k2q(q2k, bsn, nkv, bucket, nums)
        flat, lens = [], []
        B_, H_, G_, _ = offsets.shape
        for b in range(B_):
            for h in range(H_):
                for gq in range(G_):
                    for j in range(nkv):
                        r = sorted(rows[(b, h, gq, j)])
                        flat.extend(r)
                        lens.append(len(r))
        np.savez_compressed(os.path.join(HERE, name), q2k=q2k.numpy(), nums=(nums.numpy() if nums is not None else np.zeros(0, np.int32)),
                            bsn=np.array(bsn), nkv=np.array(nkv), bucket=np.array(bucket), offsets=offsets.numpy(),
                            rows_flat=np.array(flat, np.int32), rows_len=np.array(lens, np.int32))

    lit = torch.tensor([[[[0, 0, 3, -1, 9, 2], [1, 4, 4, 2, 0, 6], [2, 5, 1, 1, 3, 0], [6, 2, 3, 4, 5, 1],
                          [0, 3, 6, 6, 2, 1]],
                         [[6, 5, 4, 3, 2, 1], [0, 8, 1, 2, 3, 4], [3, 3, 3, 3, 3, 3], [1, 2, 3, 4, 5, 6],
                          [5, 0, 2, 4, 6, 1]]]], dtype=torch.int32)
    lit_nums = torch.tensor([[[5, -1, 9, 3, 1], [6, 2, 4, 5, 3]]], dtype=torch.int32)
    csr_case("csr_literal_variable.npz", lit, 0, 7, 2, lit_nums)
    g = torch.Generator().manual_seed(9)
    q2k = torch.stack([torch.randperm(23, generator=g)[:6] for _ in range(2 * 3 * 11)]).int().reshape(2, 3, 11, 6)
    csr_case("csr_random_fixed.npz", q2k, 6, 23, 4, None)
    big = (torch.arange(5 * 1025, dtype=torch.int32).reshape(1, 1, 5, 1025)) % 1103
    csr_case("csr_topk_1025.npz", big, 1025, 1103, 2, None)

    # ---------------------------------------------------------------- F. FP8 gathered reference + dequantiser
    g = torch.Generator().manual_seed(11)
    B, H, Sq, Sk = 2, 2, 200, 300
    q, k, v = rand_bf16(g, B, H, Sq, 128), rand_bf16(g, B, H, Sk, 128), rand_bf16(g, B, H, Sk, 128)
    nq, nk = 2, 3
    index = torch.stack([torch.randperm(nk, generator=g) for _ in range(B * H * nq)]).int().reshape(B, H, nq, nk)
    nums = torch.tensor([[[3, 0], [1, 2]], [[2, 3], [0, 1]]], dtype=torch.int32)
    inactive = torch.arange(nk) >= nums[..., None]
    index_p = index.masked_fill(inactive, 0x3FFFFFFF)
    sizes = torch.randint(1, 129, (B, H, nk), generator=g, dtype=torch.int32)
    sizes[..., -1].clamp_(max=Sk - (nk - 1) * 128)
    out = tf8.sparse_reference(q, k, v, index_p, nk, nums, sizes)
    q8, k8, v8, qs, ks, vs = tf8b._sage_quantize_bhsd(q, torch.nn.functional.pad(k, (0, 0, 0, 4)),
                                                      torch.nn.functional.pad(v, (0, 0, 0, 4)))
    dq_, dk_, dv_ = tf8.dequantize((q8, k8, v8, qs, ks, vs))
    np.savez_compressed(os.path.join(HERE, "fp8_gathered.npz"), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                        index=index_p.numpy(), nums=nums.numpy(), sizes=sizes.numpy(), out=out.numpy(),
                        q8=q8.view(torch.uint8).numpy(), k8=k8.view(torch.uint8).numpy(),
                        v8=v8.view(torch.uint8).numpy(), qs=qs.numpy(), ks=ks.numpy(), vs=vs.numpy(),
                        deq_q=bf16_bits(dq_), deq_k=bf16_bits(dk_), deq_v=bf16_bits(dv_))

    # ---------------------------------------------------------------- G. autograd backward reference
    g = torch.Generator().manual_seed(21)
    B, H, S = 1, 2, 384
    q, k, v, do = (rand_bf16(g, B, H, S, 128) for _ in range(4))
    index = torch.stack([torch.randperm(3, generator=g)[:2] for _ in range(B * H * 3)]).int().reshape(B, H, 3, 2)
    sizes = torch.full((3,), 128, dtype=torch.int32)
    bias = tff.block_sparse_to_attn_bias(index, 2, sizes, S, S, 128, 128)
    o, lse, dq, dk, dv = tfb._torch_ref_bwd(q, k, v, do, bias, 1.0 / math.sqrt(128), upcast=True)
    np.savez_compressed(os.path.join(HERE, "bwd_dense.npz"), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                        dout=bf16_bits(do), index=index.numpy(), out=o.float().numpy(), lse=lse.numpy(),
                        dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())

    # ---------------------------------------------------------------- G2. backward, 64-token blocks, block_sizes
    g = torch.Generator().manual_seed(22)
    B, H, Sq, Sk = 1, 2, 192, 300
    q, do = (rand_bf16(g, B, H, Sq, 128) for _ in range(2))
    k, v = (rand_bf16(g, B, H, Sk, 128) for _ in range(2))
    nq, nk = 3, 5
    index = torch.stack([torch.randperm(nk, generator=g) for _ in range(B * H * nq)]).int().reshape(B, H, nq, nk)
    nums = torch.tensor([[[3, 1, 4], [5, 2, 1]]], dtype=torch.int32)
    sizes = torch.randint(1, 65, (nk,), generator=g, dtype=torch.int32)
    sizes[-1].clamp_(max=Sk - (nk - 1) * 64)
    bias = tff.block_sparse_to_attn_bias(index, 0, sizes, Sq, Sk, 64, 64, q2k_block_nums=nums)
    o, lse, dq, dk, dv = tfb._torch_ref_bwd(q, k, v, do, bias, 1.0 / math.sqrt(128), upcast=True)
    np.savez_compressed(os.path.join(HERE, "bwd_blk64_sizes.npz"), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                        dout=bf16_bits(do), index=index.numpy(), nums=nums.numpy(), sizes=sizes.numpy(),
                        out=o.float().numpy(), lse=lse.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())

    # ---------------------------------------------------------------- I. top-k index recipe of the reference's benchmark
    # tests/bench_cutedsl_performance.py:150-167 restated with a CPU generator (the file itself draws on CUDA):
    # pooled scores ~ N(0,1) -> torch.topk(sorted=False) -> ascending sort -> int32
    g = torch.Generator().manual_seed(31)
    pooled = torch.randn(2, 3, 40, 300, generator=g)
    selected = torch.topk(pooled, 37, dim=-1, sorted=False).indices
    np.savez_compressed(os.path.join(HERE, "topk_q2k.npz"), scores=pooled.numpy(),
                        index=selected.sort(dim=-1).values.to(torch.int32).numpy())

    # ---------------------------------------------------------------- H. split policy table
    counts = [1, 2, 31, 255, 256, 449, 450, 899, 900, 2048]
    table = [ref_iface._sm100_blk64_kv_splits_from_count(c) for c in counts]
    np.savez_compressed(os.path.join(HERE, "policy_blk64_splits.npz"), counts=np.array(counts), splits=np.array(table))
    # the automatic split policy of the Sage FP8 64-token forward over a grid of (kv_blocks, heads, seqlen_q,
    # batch, num_sms) that contains every row of the table in the reference's tests/test_bsa_fp8_fwd.py:17-66
    rows = []
    for heads, seqlen_q in ((4, 64), (8, 64), (1, 64 * 37), (1, 64 * 74), (1, 64 * 100), (1, 64 * 148), (4, 119040),
                            (8, 349440), (4, 579840), (8, 695040), (4, 49290 + 2216 + 752), (2, 640), (3, 1000)):
        for kv_blocks in (1, 7, 8, 15, 16, 31, 32, 63, 64, 127, 128, 188, 255, 256, 548, 909, 915, 1089, 2048):
            for batch, num_sms in ((1, 148), (8, 148), (37, 148), (1, 200), (2, 132)):
                rows.append((kv_blocks, heads, seqlen_q, batch, num_sms,
                             ref_iface._sm100_blk64_auto_fp8_kv_splits(kv_blocks, heads, seqlen_q, batch, num_sms)))
    np.savez_compressed(os.path.join(HERE, "policy_fp8_blk64_splits.npz"), rows=np.array(rows, dtype=np.int64))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
