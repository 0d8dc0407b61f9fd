#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2|cfg2_small]

Workload (BASELINE config 2): BF16 MHA, 128-token blocks, B=2 per GPU, H=32, S=32768, D=128, every query
block keeps its diagonal KV block plus 25 uniform others (26 of 256 = 10.2 % density).  One step = one
forward (O, LSE) + one backward (k2q CSR build, preprocess, dQ, dK/dV) over that batch.  Metric:
sparse-effective TFLOPS, counting active (q block, kv block) pairs only: 4*128^2*128 FLOP per pair forward
and 10*128^2*128 backward (the reference's convention).  With N > 1 every rank owns its own batch slice
of a global batch of 2N (sharding by (batch, head), no collective on the data path): weak scaling.

The JSON line also carries: `e2e` (same metric through the public host-memory entry `HostPipeline`, pinned
host buffers, H2D of q/k/v/dO and D2H of O/LSE/dQ/dK/dV inside the timed region, head chunks pipelined over
three streams), `roofline` of the forward kernel against the
measured dense BF16 peak (MEASURED_PEAKS.json when present), `roofline_bwd`, `cpu_baseline` (the CPU
oracle on a bounded sample of the same workload, rank 0, N=1 only), `clocks` sampled with nvidia-smi
during the timed region and `gpu_launches`.

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


def run_extra(args):
    """Forward-only measurements of BASELINE configs 3, 4 and 5 on one GPU (inputs resident in HBM).
    cfg4 also times the Sage quantiser and the split-KV combine against the HBM roofline."""
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
    if args.workload == "cfg3":
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
    elif args.workload == "cfg5":
        index, nums = workloads.config5_metadata(seed=0)
        q, k, v = (rnd((4, 16, 16384, D), s) for s in (1, 2, 3))
        ic, nc = index.to(dev), nums.to(dev)
        out = torch.empty_like(q)
        ms = _time_cuda(lambda: bsa_attn_fwd(q, k, v, ic, 0, q2k_block_nums=nc, out=out, sparse_block_size=64,
                                             kv_splits="auto"), args.warmup, args.steps)
        pairs = int(nums.sum())
        tf = 4.0 * pairs * 64 * 64 * D / (ms * 1e-3) / 1e12
        # compulsory bytes: Q + O once, every active pair's K and V block through L2 (upper bound), LSE, index rows
        comp = 2 * q.numel() * 2 + pairs * 64 * 2 * D * 2 + 4 * 16 * 16384 * 4 + pairs * 4
        gbs = comp / (ms * 1e-3) / 1e9
        line.update({"value": tf, "ms_per_step": ms, "dtype": "bf16",
                     "config": {"workload": "cfg5: BF16 MHA blk64 forward, B=4 H=16 S=16384, 1% rows x 256 blocks, "
                                            "others 2-8, kv_splits=auto", "pairs": pairs},
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                                  "frac": gbs / hbm_peak, "traffic": None,
                                  "note": "compulsory bytes with every active pair's K/V counted once"},
                     "tensor_frac_of_measured": tf / bf16_peak})
    else:  # cfg4
        H, S = (4 if args.workload == "cfg4_small" else 24), 76800
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
                     "config": {"workload": f"{args.workload}: Sage FP8 blk128 forward, B=1 H={H} S=76800, band 30 + 60 far "
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
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + list(EXTRA_WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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

    # this rank's slice of the global batch (global batch = Bp * world), seeded by its global position
    g = torch.Generator().manual_seed(1000 + rank)
    host = {n: torch.randn(Bp, H, S, D, generator=g).bfloat16().pin_memory() for n in ("q", "k", "v", "do")}
    idx = make_index(Bp, H, Nq, Nq, count, 2000 + rank).to(dev)
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
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        barrier()
        e2e_ms = a.elapsed_time(b) / n_e2e
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
        peak = float(peaks.get("bf16_tflops_sustained") or peaks.get("bf16_tflops"))
        peak_burst = float(peaks.get("bf16_tflops", peak))
        step_flops = flops_f + (0 if args.fwd_only else flops_b)
        value = world * step_flops / (ms_per_step * 1e-3) / 1e12
        fwd_tf = flops_f / (fwd_ms * 1e-3) / 1e12
        bwd_tf = flops_b / (bwd_ms * 1e-3) / 1e12 if not args.fwd_only else None
        line = {
            "metric": "sparse_effective_tflops_fwd_bwd", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: BF16 MHA blk128 fwd+bwd, B={Bp}/GPU (global {Bp * world}) "
                                   f"H={H} S={S} D={D}, {count} of {Nq} KV blocks per row",
                       "pairs_per_gpu": pairs, "l2": "inputs larger than L2 (512 MiB per tensor)",
                       "sharding": "(batch, head) slices per rank, no data-path collective"},
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_tflops_per_gpu": fwd_tf, "bwd_tflops_per_gpu": bwd_tf,
            "roofline": {"bound": "tensor", "kernel": "bsa_fwd_kernel<128,bf16>", "achieved": fwd_tf, "peak": peak,
                         "peak_burst": peak_burst, "peak_source": f"{peak_kind} (sustained bf16 GEMM; kernel timed "
                         "inside a long step)", "unit": "TFLOP/s", "frac": fwd_tf / peak,
                         "frac_of_nominal_2250": fwd_tf / 2250.0,
                         # ncu dram__bytes_read+write of one forward launch on the cfg2_small capture (258 MB for
                         # 2048 query tiles), scaled by the number of tiles (profiles/cfg2_small_tcgen05_kernels.md)
                         "traffic": 258.1e6 * (Bp * H * Nq) / 2048.0 if args.workload == "cfg2" else None},
            "gpu_launches": args.steps * (1 if args.fwd_only else 9),
            "clocks": clocks,
        }
        if bwd_tf is not None:
            line["roofline_bwd"] = {"bound": "tensor", "kernel": "csr build + preprocess + bwd_dq + bwd_dkv",
                                    "achieved": bwd_tf, "peak": peak, "unit": "TFLOP/s", "frac": bwd_tf / peak,
                                    "frac_of_nominal_2250": bwd_tf / 2250.0,
                                    "note": "algorithmic 10*blk^2*D per pair; the two kernels execute 14*blk^2*D"}
        if e2e_ms is not None:
            line["e2e"] = {"value": world * step_flops / (e2e_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "ms_per_step": e2e_max, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
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
