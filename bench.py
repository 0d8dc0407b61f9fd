#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2|cfg2_small]

Workload (BASELINE config 2): BF16 MHA, 128-token blocks, B=2 per GPU, H=32, S=32768, D=128, every query
block keeps its diagonal KV block plus 25 uniform others (26 of 256 = 10.2 % density).  One step = one
forward (O, LSE) + one backward (k2q CSR build, preprocess, dQ, dK/dV) over that batch.  Metric:
sparse-effective TFLOPS, counting active (q block, kv block) pairs only: 4*128^2*128 FLOP per pair forward
and 10*128^2*128 backward (the reference's convention).  With N > 1 every rank owns its own batch slice
of a global batch of 2N (sharding by (batch, head), no collective on the data path): weak scaling.
`--no-extras` keeps only the timed step, `e2e` and `cpu_baseline`.

The JSON line also carries: `e2e` (same metric through the public host-memory entry `HostPipeline`, pinned
host buffers, H2D of q/k/v/dO and D2H of O/LSE/dQ/dK/dV inside the timed region, head chunks pipelined over
three streams, with the achieved GB/s per direction: it is PCIe-bound), `roofline` = the step's dominant
kernel (executed FLOPs / its own CUDA-event time, against the measured burst BF16 GEMM peak when the timed
region is shorter than a second, else the sustained one; `kernels` lists forward, dQ, dK/dV and preprocess),
`roofline_fwd` / `roofline_bwd` (credited FLOPs of the in-step timings), `parity` (sampled tiles of the timed
buffers against the CPU oracle), `strong_scaling` (one copy of the workload dealt by (batch, head) over the
ranks, validated through an NCCL gather of checksums), `cfg4_sage_fp8_fwd` / `cfg5_blk64_fwd` (forward-only
numbers of the other BASELINE configurations, N=1), `cpu_baseline` (the CPU oracle on a bounded sample of the
same workload, rank 0, N=1 only), `clocks` sampled with nvidia-smi during the timed region and `gpu_launches`.

`--impl reference` times the reference's CPU-runnable implementation of the path (its PyTorch masked
attention, restated in oracle/) on the host cores, on bounded samples of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "block-sparse-attention_b200"))
sys.path.insert(0, ROOT)

# forward-only lines for the other BASELINE configs; cfg4_small (4 of the 24 heads) is sized for an ncu capture
EXTRA_WORKLOADS = ("cfg3", "cfg4", "cfg4_small", "cfg5")

WORKLOADS = {
    # name: (B per GPU, H, S, blocks per row)
    "cfg2": (2, 32, 32768, 26),
    "cfg2_small": (1, 16, 16384, 13),  # same structure and density, sized for an ncu capture; never the bench line
}
BLK, D = 128, 128
# DRAM bytes (read + write) of one launch on cfg2_small (26 624 pairs), from the committed ncu capture; traffic grows
# with the number of tiles (per-tile Q / O / statistics bytes plus first-touch K / V), so it is scaled by the pairs
NCU_SMALL_PAIRS = 26624
NCU_DRAM_BYTES_SMALL = {"bsa_fwd_kernel<128,bf16>": 248.7e6, "bwd_dq_kernel<128>": 324.2e6, "bwd_dkv_kernel<128>": 381.1e6}
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def make_index(B, H, Nq, Nkv, count, seed):
    """diagonal + (count-1) distinct uniform others per row, ascending int32 - vectorised."""
    g = torch.Generator().manual_seed(seed)
    keys = torch.rand(B, H, Nq, Nkv, generator=g)
    diag = torch.arange(Nq).clamp(max=Nkv - 1)
    keys[..., torch.arange(Nq), diag] = -1.0  # the diagonal always wins
    idx = keys.argsort(dim=-1)[..., :count]
    return idx.sort(dim=-1).values.to(torch.int32).contiguous()


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampling during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        busy = [x for x in sm if x > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_sample(B, H, S, count, seed, heads, do_bwd=True):
    """CPU oracle (gathered fp32 attention + its backward) on `heads` heads of batch 0; returns
    (pairs, seconds_fwd, seconds_bwd)."""
    from oracle import bsa_oracle as orc
    Nq = S // BLK
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, heads, S, D, generator=g).bfloat16()
    k = torch.randn(1, heads, S, D, generator=g).bfloat16()
    v = torch.randn(1, heads, S, D, generator=g).bfloat16()
    do = torch.randn(1, heads, S, D, generator=g).bfloat16()
    idx = make_index(1, heads, Nq, Nq, count, seed)
    t0 = time.perf_counter()
    orc.attention_gathered(q, k, v, idx, count, blk=BLK)
    t1 = time.perf_counter()
    tb = 0.0
    if do_bwd:
        orc.backward_gathered(q, k, v, do, idx, count, blk=BLK)
        tb = time.perf_counter() - t1
    return heads * Nq * count, t1 - t0, tb


def run_reference(args, rank, world):
    if rank != 0:
        return
    Bp, H, S, count = WORKLOADS[args.workload]
    torch.set_num_threads(os.cpu_count() or 1)
    heads = 8
    times = []
    for i in range(args.warmup + args.steps):
        pairs, tf, tb = cpu_sample(Bp, H, S, count, 100 + i, heads)
        if i >= args.warmup:
            times.append((tf, tb))
    tf = sum(t[0] for t in times) / len(times)
    tb = sum(t[1] for t in times) / len(times)
    flops = (4 + 10) * pairs * BLK * BLK * D
    val = flops / (tf + tb) / 1e12
    sample = f"{heads} of {Bp * H} (batch, head) slices per step, all {S // BLK} query tiles, forward + backward"
    line = {
        "impl": "reference", "metric": "sparse_effective_tflops_fwd_bwd", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": (tf + tb) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: BF16-valued inputs, B={Bp}/GPU H={H} S={S} D={D} blk128 "
                               f"{count} blocks/row; CPU arm computes a bounded sample in fp32"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample, "fwd_tflops": 4 * pairs * BLK * BLK * D / tf / 1e12,
                         "bwd_tflops": 10 * pairs * BLK * BLK * D / tb / 1e12},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _time_cuda(fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in evs)


def run_extra(args, workload=None, emit=True):
    """Forward-only measurements of BASELINE configs 3, 4 and 5 on one GPU (inputs resident in HBM).
    cfg4 also times the Sage quantiser and the split-KV combine against the HBM roofline.  Returns the line."""
    workload = workload or args.workload
    from block_sparse_attention import (bsa_attn_fwd, bsa_fp8_blk128_fwd, check_device_status,
                                        quantize_sage_bhsd)
    from oracle import workloads
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_kind = load_peaks()
    bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))

    def rnd(shape, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.randn(shape, generator=g, device=dev).to(torch.bfloat16)

    line = {"metric": "sparse_effective_tflops_fwd", "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "data": "synthetic", "peak_source": peak_kind}
    if workload == "cfg3":
        index, nums = workloads.config3_metadata(seed=0)
        q, k, v = rnd((1, 64, 65536, D), 1), rnd((1, 8, 65536, D), 2), rnd((1, 8, 65536, D), 3)
        ic, nc = index.to(dev), nums.to(dev)
        out = torch.empty_like(q)
        ms = _time_cuda(lambda: bsa_attn_fwd(q, k, v, ic, 0, q2k_block_nums=nc, pack_gqa=True, out=out,
                                             sparse_block_size=128), args.warmup, args.steps)
        pairs = int(nums.sum())
        tf = 4.0 * pairs * 128 * 128 * D / (ms * 1e-3) / 1e12
        line.update({"value": tf, "ms_per_step": ms, "dtype": "bf16",
                     "config": {"workload": "cfg3: BF16 GQA blk128 forward, B=1 Hq=64 Hkv=8 pack_gqa S=65536, "
                                            "Poisson(25) blocks per packed tile, 2% empty", "pairs": pairs},
                     "roofline": {"bound": "tensor", "achieved": tf, "peak": bf16_peak, "unit": "TFLOP/s",
                                  "frac": tf / bf16_peak, "frac_of_nominal_2250": tf / 2250.0, "traffic": None}})
    elif workload == "cfg5":
        index, nums = workloads.config5_metadata(seed=0)
        q, k, v = (rnd((4, 16, 16384, D), s) for s in (1, 2, 3))
        ic, nc = index.to(dev), nums.to(dev)
        out = torch.empty_like(q)
        ms = _time_cuda(lambda: bsa_attn_fwd(q, k, v, ic, 0, q2k_block_nums=nc, out=out, sparse_block_size=64,
                                             kv_splits="auto"), args.warmup, args.steps)
        pairs = int(nums.sum())
        tf = 4.0 * pairs * 64 * 64 * D / (ms * 1e-3) / 1e12
        # compulsory HBM bytes: Q and O once, LSE, the index rows, and the K / V blocks that are touched at all
        # (first touch; the re-reads of a block by other query tiles are L2 traffic, reported separately)
        live = torch.arange(index.shape[-1])[None, None, None, :] < nums[..., None]
        touched = torch.zeros(4, 16, 256, dtype=torch.bool)
        bi, hi, _, _ = torch.nonzero(live, as_tuple=True)
        touched[bi, hi, index[live].long()] = True
        kv_unique = int(touched.sum()) * 64 * 2 * D * 2
        comp = 2 * q.numel() * 2 + kv_unique + 4 * 16 * 16384 * 4 + pairs * 4 + nums.numel() * 4
        l2_side = 2 * q.numel() * 2 + pairs * 64 * 2 * D * 2 + 4 * 16 * 16384 * 4 + pairs * 4
        gbs = comp / (ms * 1e-3) / 1e9
        line.update({"value": tf, "ms_per_step": ms, "dtype": "bf16",
                     "config": {"workload": "cfg5: BF16 MHA blk64 forward, B=4 H=16 S=16384, 1% rows x 256 blocks, "
                                            "others 2-8, kv_splits=auto", "pairs": pairs},
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                                  "frac": gbs / hbm_peak, "traffic": None, "compulsory_bytes": comp,
                                  "note": "compulsory bytes: Q + O + LSE + index + first-touch K/V blocks"},
                     "l2_side_gbs": l2_side / (ms * 1e-3) / 1e9,
                     "l2_side_note": "every active pair's K/V block counted (what L2 must deliver)",
                     "tensor_frac_of_measured": tf / bf16_peak})
    else:  # cfg4
        H, S = (4 if workload == "cfg4_small" else 24), 76800
        index, nums = workloads.config4_metadata(seed=0, heads=H)
        q = rnd((1, H, S, D), 1)
        k = workloads.k_with_channel_bias((1, H, S, D), 2, dev)
        v = rnd((1, H, S, D), 3)
        ic, nc = index.to(dev), nums.to(dev)
        ms_quant = _time_cuda(lambda: quantize_sage_bhsd(q, k, v), args.warmup, args.steps)
        quant = quantize_sage_bhsd(q, k, v)
        ms4 = _time_cuda(lambda: bsa_fp8_blk128_fwd(*quant, ic, 0, q2k_block_nums=nc, kv_splits=4),
                         args.warmup, args.steps)
        ms1 = _time_cuda(lambda: bsa_fp8_blk128_fwd(*quant, ic, 0, q2k_block_nums=nc, kv_splits=1),
                         args.warmup, args.steps)
        pairs = int(nums.sum())
        flops = 4.0 * pairs * 128 * 128 * D
        tf4, tf1 = flops / (ms4 * 1e-3) / 1e12, flops / (ms1 * 1e-3) / 1e12
        fp8_peak = 2.0 * bf16_peak  # no FP8 GEMM peak is measured: twice the measured BF16 figure (assumption)
        n = q.numel()
        quant_bytes = 3 * n + 5 * n + 5 * n
        line.update({"value": tf4, "ms_per_step": ms4, "dtype": "e4m3",
                     "config": {"workload": f"{workload}: Sage FP8 blk128 forward, B=1 H={H} S=76800, band 30 + 60 far "
                                            "blocks (19.9% density), kv_splits=4 incl. combine", "pairs": pairs},
                     "unsplit_ms": ms1, "unsplit_tflops": tf1,
                     "roofline": {"bound": "tensor", "achieved": tf4, "peak": fp8_peak, "unit": "TFLOP/s",
                                  "frac": tf4 / fp8_peak, "frac_of_nominal_4500": tf4 / 4500.0, "traffic": None,
                                  "note": "FP8 peak taken as 2x the measured BF16 GEMM peak"},
                     "quantiser": {"ms": ms_quant, "bound": "hbm", "achieved": quant_bytes / (ms_quant * 1e-3) / 1e9,
                                   "peak": hbm_peak, "unit": "GB/s",
                                   "frac": quant_bytes / (ms_quant * 1e-3) / 1e9 / hbm_peak,
                                   "bytes": "3|Q| + 5|K| + 5|V|"}})
    check_device_status()
    if emit:
        print(json.dumps(line), flush=True)
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + list(EXTRA_WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the per-kernel, strong-scaling, cfg4 / cfg5 and parity legs behind the timed region")
    ap.add_argument("--fwd-only", action="store_true", help="profiling aid: skip the backward pass")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.fwd_only else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.workload in EXTRA_WORKLOADS:
        if rank == 0:
            run_extra(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the engine has no CPU path")
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd, check_device_status
    from block_sparse_attention.bsa_attn_interface import _bsa_attn_bwd
    from block_sparse_attention.sharding import gather_slices, shard_batch_heads, sharded_fwd_bwd

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    Bp, H, S, count = WORKLOADS[args.workload]
    Nq = S // BLK
    pairs = Bp * H * Nq * count
    flops_f = 4.0 * pairs * BLK * BLK * D
    flops_b = 10.0 * pairs * BLK * BLK * D

    # Weak scaling: every rank owns one batch slice (B = Bp) of a global batch Bp * world.  All slices hold the
    # same seeded values, so that the strong-scaling leg below can check a rank's shard against rank 0's copy.
    g = torch.Generator().manual_seed(1000)
    host = {n: torch.randn(Bp, H, S, D, generator=g).bfloat16().pin_memory() for n in ("q", "k", "v", "do")}
    idx_host = make_index(Bp, H, Nq, Nq, count, 2000)
    idx = idx_host.to(dev)
    q, k, v, do = (host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "do"))
    out = torch.empty_like(q)
    lse = torch.empty(Bp, H, S, dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    torch.cuda.synchronize()

    def step(ev=None):
        if ev:
            ev[0].record()
        bsa_attn_fwd(q, k, v, idx, count, out=out, lse=lse, sparse_block_size=BLK)
        if ev:
            ev[1].record()
        if not args.fwd_only:
            bsa_attn_bwd(do, q, k, v, out, lse, idx, count, dq=dq, dk=dk, dv=dv, sparse_block_size=BLK)
        if ev:
            ev[2].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    check_device_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record()
    for i in range(args.steps):
        step(evs[i])
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    check_device_status()
    total_ms = t_begin.elapsed_time(t_end)
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)

    # ---- the kernels of the step one by one: the same step with the backward issued as its three passes, CUDA events
    # between them (same buffers, same order and duty cycle as the timed step, so clocks and caches are comparable)
    kernels = None
    if not args.no_extras and not args.fwd_only:
        n_k = max(3, min(args.steps, 10))

        def bwd_stage(mask):
            _bsa_attn_bwd(do, q, k, v, out, lse, idx, count, dq=dq, dk=dk, dv=dv, sparse_block_size=BLK, stages=mask)
        bwd_stage(7)  # fills the row statistics the single passes read
        split_evs = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(n_k)]
        for ev in split_evs:
            ev[0].record()
            bsa_attn_fwd(q, k, v, idx, count, out=out, lse=lse, sparse_block_size=BLK)
            ev[1].record()
            bwd_stage(1)
            ev[2].record()
            bwd_stage(2)
            ev[3].record()
            bwd_stage(4)
            ev[4].record()
        torch.cuda.synchronize()
        names = ("fwd", "bwd_preprocess", "bwd_dq", "bwd_dkv")
        kernels = {n: statistics.median(ev[i].elapsed_time(ev[i + 1]) for ev in split_evs) for i, n in enumerate(names)}
        check_device_status()

    # ---- parity of what was timed: sampled tiles of O / LSE / dQ against the CPU oracle (rank 0)
    parity = None
    if rank == 0 and not args.no_extras and not args.fwd_only:
        from oracle import bsa_oracle as orc
        torch.cuda.synchronize()
        parity = {"max_abs_O": 0.0, "max_abs_LSE": 0.0, "max_abs_dQ": 0.0, "tiles": []}
        for (b, h, m) in ((0, 0, 0), (Bp - 1, H - 1, Nq - 1)):
            rows = slice(m * BLK, (m + 1) * BLK)
            qs, dos = host["q"][b:b + 1, h:h + 1, rows], host["do"][b:b + 1, h:h + 1, rows]
            ks, vs = host["k"][b:b + 1, h:h + 1], host["v"][b:b + 1, h:h + 1]
            ix = idx_host[b:b + 1, h:h + 1, m:m + 1]
            ro, rl = orc.attention_gathered(qs, ks, vs, ix, count, blk=BLK)
            rdq, _, _ = orc.backward_gathered(qs, ks, vs, dos, ix, count, blk=BLK)
            parity["max_abs_O"] = max(parity["max_abs_O"], (out[b, h, rows].float().cpu() - ro[0, 0]).abs().max().item())
            parity["max_abs_LSE"] = max(parity["max_abs_LSE"], (lse[b, h, rows].cpu() - rl[0, 0]).abs().max().item())
            parity["max_abs_dQ"] = max(parity["max_abs_dQ"], (dq[b, h, rows].float().cpu() - rdq[0, 0]).abs().max().item())
            parity["tiles"].append([b, h, m])
        parity["tolerance"] = {"O": 3e-2, "LSE": 2e-3, "dQ": "3*|bf16 - fp32| + 3*eps + 5e-3 (about 2e-2)"}
        parity["ok"] = parity["max_abs_O"] <= 3e-2 and parity["max_abs_LSE"] <= 2e-3 and parity["max_abs_dQ"] <= 5e-2

    # ---- strong scaling: ONE copy of the workload, its Bp * H (batch, head) slices dealt over the ranks
    strong = None
    if not args.no_extras and not args.fwd_only:
        mine = shard_batch_heads(Bp, H, world, rank)
        buf = {"q": gather_slices(q, mine), "k": gather_slices(k, mine), "v": gather_slices(v, mine),
               "dout": gather_slices(do, mine), "index": gather_slices(idx, mine).contiguous()}
        for n in ("out", "dq", "dk", "dv"):
            buf[n] = torch.empty_like(buf["q"])
        buf["lse"] = torch.empty(1, len(mine), S, dtype=torch.float32, device=dev)
        res = sharded_fwd_bwd(None, None, None, None, None, count, mine, BLK, buffers=buf)
        barrier()
        n_s = max(3, min(args.steps, 10))
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_s):
            res = sharded_fwd_bwd(None, None, None, None, None, count, mine, BLK, buffers=buf)
        b_.record()
        barrier()
        check_device_status()
        strong_ms = a.elapsed_time(b_) / n_s
        # the shard must be bit-identical to the same slices of this rank's unsharded results ...
        same = all(torch.equal(res[n][0, i], full[b, h]) for i, (b, h) in enumerate(mine)
                   for n, full in (("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)))
        # ... and, gathered over NCCL (validation only), to rank 0's copy of every slice
        sums = torch.zeros(Bp * H, 5, dtype=torch.float64, device=dev)
        for i, (b, h) in enumerate(mine):
            for j, n in enumerate(("out", "lse", "dq", "dk", "dv")):
                sums[b * H + h, j] = res[n][0, i].double().sum()
        st = torch.tensor([strong_ms, 0.0 if same else 1.0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(sums)  # shards are disjoint: the sum is the gather
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        if rank == 0:
            ref_sums = torch.stack([torch.stack([t[b, h].double().sum() for t in (out, lse, dq, dk, dv)])
                                    for b in range(Bp) for h in range(H)])
            strong_ms_max = st[0].item()
            strong = {
                "scaling": "strong", "workload": f"one copy of {args.workload}: {Bp * H} (batch, head) slices, "
                                                 f"{len(mine)} per rank, fwd+bwd", "ms_per_step": strong_ms_max,
                "tflops_total": (flops_f + flops_b) / (strong_ms_max * 1e-3) / 1e12,
                "tflops_per_gpu": (flops_f + flops_b) / (strong_ms_max * 1e-3) / 1e12 / world,
                "shards_bit_identical_to_unsharded": st[1].item() == 0.0,
                "gathered_checksums_match_rank0": bool(torch.equal(sums, ref_sums)),
                "collective": "NCCL all_reduce of per-slice checksums after the timed region (validation only)",
            }
        del buf, res

    # ---- end-to-end through the public API with host buffers
    e2e = None
    if not args.no_e2e and not args.fwd_only:
        host_out = {n: torch.empty(Bp, H, S, D, dtype=torch.bfloat16).pin_memory() for n in ("o", "dq", "dk", "dv")}
        host_lse = torch.empty(Bp, H, S, dtype=torch.float32).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = sum(t.numel() * t.element_size() for t in host_out.values()) + host_lse.numel() * 4

        from block_sparse_attention.host_pipeline import HostPipeline
        # the public host-memory entry: head chunks pipelined over copy / compute / copy streams.  Two heads per
        # chunk: the first copy in and the last copy out are the only ones nothing overlaps, so short chunks win
        # until the per-chunk launches dominate (8 / 4 / 2 / 1 heads: 52.8 / 51.0 / 48.4 / 51.1 ms on this shape)
        pipe = HostPipeline(Bp, H, S, S, idx, count, heads_per_chunk=2)
        host_res = {"out": host_out["o"], "lse": host_lse, "dq": host_out["dq"], "dk": host_out["dk"],
                    "dv": host_out["dv"]}
        host_src = {"q": host["q"], "k": host["k"], "v": host["v"], "dout": host["do"]}

        def e2e_step():
            pipe.run(host_src, host_res)

        e2e_step()
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b_.record()
        barrier()
        e2e_ms = a.elapsed_time(b_) / n_e2e
    else:
        e2e_ms, h2d, d2h = None, 0, 0

    # ---- max over ranks
    stats = torch.tensor([total_ms, fwd_ms, bwd_ms, e2e_ms or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms, e2e_max = stats.tolist()
    ms_per_step = total_ms / args.steps

    if rank == 0:
        peaks, peak_kind = load_peaks()
        peak_burst = float(peaks.get("bf16_tflops") or FALLBACK_PEAKS["bf16_tflops"])
        peak_sust = float(peaks.get("bf16_tflops_sustained") or peak_burst)
        hbm_peak = float(peaks.get("hbm_gbs") or FALLBACK_PEAKS["hbm_gbs"])
        # a timed region of less than a second is compared with the burst GEMM figure, a longer one with the
        # sustained one; both fractions are in the line.  (The power cap is active within about ten launches of
        # these kernels - see `clocks` - so the burst figure is the stricter of the two here.)
        timed_s = total_ms * 1e-3
        peak = peak_burst if timed_s < 1.0 else peak_sust
        peak_name = "burst" if timed_s < 1.0 else "sustained"
        step_flops = flops_f + (0 if args.fwd_only else flops_b)
        value = world * step_flops / (ms_per_step * 1e-3) / 1e12
        fwd_tf = flops_f / (fwd_ms * 1e-3) / 1e12
        bwd_tf = flops_b / (bwd_ms * 1e-3) / 1e12 if not args.fwd_only else None
        unit = pairs * BLK * BLK * D / 1e12  # TFLOP per "1 * blk^2 * D" of every pair

        def entry(name, ms, credited, executed, where):
            ach_c, ach_e = credited * unit / (ms * 1e-3), executed * unit / (ms * 1e-3)
            return {"kernel": name, "ms": ms, "timed": where, "credited_tflops": ach_c, "executed_tflops": ach_e,
                    "frac_credited": ach_c / peak, "frac_executed": ach_e / peak,
                    "frac_executed_of_burst": ach_e / peak_burst,
                    "frac_credited_of_nominal_2250": ach_c / 2250.0}
        per_kernel = [entry("bsa_fwd_kernel<128,bf16>", fwd_ms, 4, 4, "inside the step")]
        if kernels is not None:
            # credited work of the backward (10 per pair) split by the GEMMs a kernel contributes: dQ kernel
            # S, dP, dQ (executes 6, credited 4: dQ = 2 plus half of the shared S and dP), dK/dV kernel S^T, dP^T,
            # dV, dK (executes 8, credited 6)
            per_kernel += [entry("bsa_fwd_kernel<128,bf16>", kernels["fwd"], 4, 4, "inside a split step"),
                           entry("bwd_dq_kernel<128>", kernels["bwd_dq"], 4, 6, "inside a split step (csr build included)"),
                           entry("bwd_dkv_kernel<128>", kernels["bwd_dkv"], 6, 8, "inside a split step (csr build included)")]
        dominant = max(per_kernel[1:] or per_kernel, key=lambda e: e["ms"])
        line = {
            "metric": "sparse_effective_tflops_fwd_bwd", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: BF16 MHA blk128 fwd+bwd, B={Bp}/GPU (global {Bp * world}) "
                                   f"H={H} S={S} D={D}, {count} of {Nq} KV blocks per row",
                       "pairs_per_gpu": pairs, "l2": "inputs larger than L2 (512 MiB per tensor)",
                       "sharding": "(batch, head) slices per rank, no data-path collective"},
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_tflops_per_gpu": fwd_tf, "bwd_tflops_per_gpu": bwd_tf,
            "roofline": {"bound": "tensor", "kernel": dominant["kernel"], "timed": dominant["timed"],
                         "achieved": dominant["executed_tflops"], "achieved_credited": dominant["credited_tflops"],
                         "peak": peak, "peak_kind": f"{peak_kind} {peak_name} bf16 GEMM "
                         f"(timed region {timed_s:.2f} s)", "peak_burst": peak_burst, "peak_sustained": peak_sust,
                         "unit": "TFLOP/s", "frac": dominant["executed_tflops"] / peak,
                         "frac_credited": dominant["credited_tflops"] / peak,
                         "frac_of_burst": dominant["executed_tflops"] / peak_burst,
                         "frac_of_sustained": dominant["executed_tflops"] / peak_sust,
                         "frac_of_nominal_2250": dominant["executed_tflops"] / 2250.0,
                         "traffic": None,
                         "traffic_from_profile": {
                             "bytes_per_launch_scaled": NCU_DRAM_BYTES_SMALL.get(dominant["kernel"], 0) * (pairs / NCU_SMALL_PAIRS),
                             "file": "profiles/cfg2_small_tcgen05_kernels.md",
                             "how": "dram__bytes_read + write of one launch in the ncu capture of cfg2_small, scaled "
                                    "by the number of pairs; not measured by this run"},
                         "note": "achieved = FLOPs the kernel executes / its CUDA-event time; 'credited' scales it "
                                 "to the metric's 4 (fwd) / 10 (bwd) * blk^2 * D per pair",
                         "kernels": per_kernel},
            "roofline_fwd": {"bound": "tensor", "achieved": fwd_tf, "peak": peak, "frac": fwd_tf / peak,
                             "frac_of_nominal_2250": fwd_tf / 2250.0, "unit": "TFLOP/s"},
            "gpu_launches": args.steps * (1 if args.fwd_only else 9),
            "clocks": clocks,
        }
        if bwd_tf is not None:
            line["roofline_bwd"] = {"bound": "tensor", "kernel": "csr build + preprocess + bwd_dq + bwd_dkv",
                                    "achieved": bwd_tf, "peak": peak, "unit": "TFLOP/s", "frac": bwd_tf / peak,
                                    "frac_of_nominal_2250": bwd_tf / 2250.0,
                                    "note": "algorithmic 10*blk^2*D per pair; the two kernels execute 14*blk^2*D"}
        if kernels is not None:
            pre_bytes = 2 * q.numel() * 2 + 3 * lse.numel() * 4
            line["roofline"]["kernels"].append(
                {"kernel": "bwd_preprocess_kernel", "ms": kernels["bwd_preprocess"], "timed": "inside a split step (csr build included)",
                 "bound": "hbm", "achieved_gbs": pre_bytes / (kernels["bwd_preprocess"] * 1e-3) / 1e9,
                 "frac": pre_bytes / (kernels["bwd_preprocess"] * 1e-3) / 1e9 / hbm_peak})
        if parity is not None:
            line["parity"] = parity
            line["max_abs_O"], line["max_abs_dQ"] = parity["max_abs_O"], parity["max_abs_dQ"]
        if strong is not None:
            line["strong_scaling"] = strong
        if e2e_ms is not None:
            line["e2e"] = {"value": world * step_flops / (e2e_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "ms_per_step": e2e_max, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "bound": "pcie", "h2d_gbs_per_gpu": h2d / (e2e_max * 1e-3) / 1e9,
                           "d2h_gbs_per_gpu": d2h / (e2e_max * 1e-3) / 1e9,
                           "note": "both directions run concurrently; a step costs about max(H2D, D2H, compute)"}
        if world == 1 and not args.no_extras and not args.fwd_only:
            # the other BASELINE configurations, forward only, a few seconds each
            del q, k, v, do, out, lse, dq, dk, dv
            torch.cuda.empty_cache()
            ex_args = argparse.Namespace(steps=max(3, min(args.steps, 10)), warmup=3)
            c4, c5 = run_extra(ex_args, "cfg4", emit=False), run_extra(ex_args, "cfg5", emit=False)
            line["cfg4_sage_fp8_fwd"] = {k_: c4[k_] for k_ in ("value", "ms_per_step", "unsplit_ms", "unsplit_tflops",
                                                              "roofline", "quantiser", "config")}
            line["cfg4_sage_fp8_fwd"]["roofline_unsplit"] = {
                "achieved": c4["unsplit_tflops"], "peak": c4["roofline"]["peak"],
                "frac": c4["unsplit_tflops"] / c4["roofline"]["peak"],
                "frac_of_nominal_4500": c4["unsplit_tflops"] / 4500.0}
            line["cfg5_blk64_fwd"] = {k_: c5[k_] for k_ in ("value", "ms_per_step", "roofline", "l2_side_gbs", "config")}
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            n_heads = min(H, 32)
            cp, tf, tb = cpu_sample(Bp, H, S, count, 7, heads=n_heads)
            line["cpu_baseline"] = {
                "value": (4 + 10) * cp * BLK * BLK * D / (tf + tb) / 1e12, "unit": "TFLOP/s",
                "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"{n_heads} of {Bp * H} (batch, head) slices, all {Nq} query tiles, "
                          f"fwd {tf:.2f} s + bwd {tb:.2f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
