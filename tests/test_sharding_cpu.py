"""CPU: (batch, head) sharding logic, single process and world_size-2 gloo."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from block_sparse_attention.sharding import flat_slices, shard_batch_heads
from oracle import bsa_oracle as orc


def test_partition_is_exact():
    for B, H, W in [(2, 32, 8), (1, 8, 8), (1, 24, 8), (4, 16, 3), (1, 3, 4)]:
        seen = []
        for r in range(W):
            seen += shard_batch_heads(B, H, W, r)
        assert sorted(seen) == flat_slices(B, H)
    w = [float(i % 5 + 1) for i in range(12)]
    loads = []
    seen = []
    for r in range(4):
        mine = shard_batch_heads(3, 4, 4, r, weights=w)
        seen += mine
        loads.append(sum(w[b * 4 + h] for b, h in mine))
    assert sorted(seen) == flat_slices(3, 4)
    assert max(loads) - min(loads) <= max(w)


def _worker(rank, world, port, q, k, v, index, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, H = q.shape[:2]
    out = torch.zeros_like(q, dtype=torch.float32)
    for b, h in shard_batch_heads(B, H, world, rank):
        o, _ = orc.attention_gathered(q, k, v, index, 2, heads=[h], batches=[b])
        out[b, h] = o[b, h]
    dist.all_reduce(out)  # validation-only collective: shards are disjoint, so the sum is the gather
    if rank == 0:
        ret.put(out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_sharded_forward_matches_single_process():
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 4, 256, 128, generator=gen) for _ in range(3))
    index = orc.make_uniform_index(1, 4, 2, 2, 2, gen)
    full, _ = orc.attention_gathered(q, k, v, index, 2)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, k, v, index, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert torch.allclose(got, full, atol=1e-6)
