#!/usr/bin/env python
"""Per-role phase table of the tcgen05 kernels (development tool).

    python build.py --phase-timers
    python phase_timers.py [--workload cfg2_small|cfg2|cfg4_small] [--lib PATH]

Loads the instrumented library (``libbsa_b200_timers.so``: lane 0 of one warp per role accumulates
``clock64()`` deltas per phase, summed over all CTAs), runs the forward and the backward of the workload
a few times and prints, for every role, the clocks per active (q block, kv block) pair of one CTA.  All
rows of one kernel add up to about the same total: the kernel's clocks per pair of one CTA (the forward runs
two CTAs per SM, so an SM spends half of that per pair).  The numbers are taken
with the timers compiled in, which costs a few percent; they locate waits, they are not bench values.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

FWD_ROLES = {"softmax warps": 0, "MMA issuer": 32, "TMA producer": 48}
FWD_PHASES = {
    "softmax": ["other", "wait S", "tmem ld + first max", "max + rescale", "exp + P store", "st wait + arrive",
                "epilogue: wait O", "epilogue: scale + store"],
    "issuer": ["other", "wait Q", "wait K", "wait V", "wait P", "-", "issue PV", "issue QK"],
    "producer": ["other", "wait Q free", "wait ring free", "-", "-", "-", "-", "-"],
}
BWD_ROLES = {
    "dQ compute group 0": 0, "dQ compute group 1": 8, "dQ issuer S": 16, "dQ issuer dQ": 24, "dQ issuer dP": 32,
    "dK/dV compute group 0": 64, "dK/dV compute group 1": 72, "dK/dV issuer 0 (S^T, dV)": 80,
    "dK/dV issuer 1 (dP^T, dK)": 88, "dK/dV producer": 96,
}
BWD_PHASES = {
    "dq_compute": ["other", "wait S", "ld S + exp", "wait dP", "ld dP + dS + st", "epilogue", "-", "-"],
    "dq_issuer": ["other + issue", "wait Q / dO", "wait ring", "wait dS / dS-used", "wait dQ free", "wait S free",
                  "-", "-"],
    "dkv_compute": ["other", "wait S^T", "ld S^T + exp", "wait dP^T", "dS^T + st", "epilogue",
                    "ld dP^T + P^T st", "wait row stats"],
    "dkv_issuer": ["other", "wait Q tile", "wait dO tile", "wait S free / dV done", "wait P^T / dS^T", "issue S^T / dK", "issue dV",
                   "issue dP^T"],
    "dkv_producer": ["other + issue", "wait K/V free", "wait stage for Q", "wait stage for dO", "-", "-", "-", "-"],
}


def table(title, roles, counters, phases_of, pairs_per_cta):
    print(f"\n{title}  (clocks per active pair of one CTA)")
    for name, base in roles.items():
        vals = [counters[base + i] / pairs_per_cta for i in range(8)]
        labels = phases_of(name)
        cells = ", ".join(f"{lab} {v:.0f}" for lab, v in zip(labels, vals) if lab != "-" and v >= 0.5)
        print(f"  {name:32s} total {sum(vals):6.0f}: {cells}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2_small", choices=["cfg2_small", "cfg2", "cfg4_small"])
    ap.add_argument("--lib", default=os.path.join(HERE, "block_sparse_attention", "libbsa_b200_timers.so"))
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    os.environ["BSA_B200_LIB"] = args.lib
    sys.path.insert(0, HERE)
    import torch
    from block_sparse_attention import _cabi, bsa_attn_bwd, bsa_attn_fwd, bsa_fp8_blk128_fwd, quantize_sage_bhsd

    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    fwd_buf = (ctypes.c_ulonglong * 64)()
    bwd_buf = (ctypes.c_ulonglong * 128)()
    lib.bsa_fwd_phase_timers.argtypes = [ctypes.c_void_p]
    lib.bsa_bwd_phase_timers.argtypes = [ctypes.c_void_p]
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape):
        return torch.randn(shape, generator=g, device=dev).to(torch.bfloat16)

    if args.workload == "cfg4_small":
        B, H, S, band, far = 1, 4, 76800, 30, 60
        Nq = S // 128
        # band of +-30 blocks plus 60 far blocks per row (the video-DiT-like pattern), ascending
        keys = torch.rand(B, H, Nq, Nq, generator=g, device=dev)
        i = torch.arange(Nq, device=dev)
        near = (i[:, None] - i[None, :]).abs() <= band
        keys = torch.where(near, torch.full_like(keys, -1.0), keys)
        nums = (near.sum(-1).to(torch.int32) + far)[None, None].expand(B, H, Nq).contiguous()
        idx = keys.argsort(dim=-1)[..., :int(nums.max())].to(torch.int32).contiguous()
        q, k, v = rnd(B, H, S, 128), rnd(B, H, S, 128), rnd(B, H, S, 128)
        quant = quantize_sage_bhsd(q, k, v)
        pairs = int(nums.sum())
        lib.bsa_fwd_phase_timers(fwd_buf)
        for _ in range(args.iters):
            bsa_fp8_blk128_fwd(*quant, idx, 0, q2k_block_nums=nums, kv_splits=1)
        lib.bsa_fwd_phase_timers(fwd_buf)
        per_cta = pairs * args.iters  # the counters are sums over all CTAs
        table(f"Sage FP8 forward, {args.workload} ({pairs} pairs)", FWD_ROLES, list(fwd_buf),
              lambda n: FWD_PHASES["softmax" if n.startswith("softmax") else "issuer" if n.startswith("MMA") else "producer"],
              per_cta)
        return

    B, H, S, count = (2, 32, 32768, 26) if args.workload == "cfg2" else (1, 16, 16384, 13)
    Nq = S // 128
    keys = torch.rand(B, H, Nq, Nq, generator=g, device=dev)
    keys[..., torch.arange(Nq), torch.arange(Nq)] = -1.0
    idx = keys.argsort(dim=-1)[..., :count].sort(dim=-1).values.to(torch.int32).contiguous()
    q, k, v, do = rnd(B, H, S, 128), rnd(B, H, S, 128), rnd(B, H, S, 128), rnd(B, H, S, 128)
    out = torch.empty_like(q)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=dev)
    pairs = B * H * Nq * count
    per_cta = pairs * args.iters  # the counters are sums over all CTAs
    lib.bsa_fwd_phase_timers(fwd_buf)
    lib.bsa_bwd_phase_timers(bwd_buf)
    for _ in range(args.iters):
        bsa_attn_fwd(q, k, v, idx, count, out=out, lse=lse, sparse_block_size=128)
    lib.bsa_fwd_phase_timers(fwd_buf)
    for _ in range(args.iters):
        bsa_attn_bwd(do, q, k, v, out, lse, idx, count, sparse_block_size=128)
    lib.bsa_bwd_phase_timers(bwd_buf)
    table(f"BF16 forward, {args.workload} ({pairs} pairs)", FWD_ROLES, list(fwd_buf),
          lambda n: FWD_PHASES["softmax" if n.startswith("softmax") else "issuer" if n.startswith("MMA") else "producer"],
          per_cta)

    def bwd_phases(n):
        if n.startswith("dQ compute"):
            return BWD_PHASES["dq_compute"]
        if n.startswith("dQ issuer"):
            return BWD_PHASES["dq_issuer"]
        if n.startswith("dK/dV compute"):
            return BWD_PHASES["dkv_compute"]
        if n.startswith("dK/dV producer"):
            return BWD_PHASES["dkv_producer"]
        return BWD_PHASES["dkv_issuer"]

    table(f"BF16 backward, {args.workload} ({pairs} pairs)", BWD_ROLES, list(bwd_buf), bwd_phases, per_cta)


if __name__ == "__main__":
    main()
