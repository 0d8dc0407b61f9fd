"""GPU: the (batch, head) sharding helper on the product path.  The slices a rank owns are gathered into one
[1, n, S, D] problem; every slice must come out bit-identical to the same slice of the unsharded call, whatever the
partition (this is what lets ranks work without any collective on the data path)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sharded_slices_are_bit_identical_to_the_unsharded_call():
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd
    from block_sparse_attention.sharding import shard_batch_heads, sharded_fwd_bwd
    from oracle import bsa_oracle as orc
    gen = torch.Generator().manual_seed(3)
    B, H, S, count = 2, 3, 1024, 3
    q, k, v, do = (torch.randn(B, H, S, 128, generator=gen).bfloat16().cuda() for _ in range(4))
    index = orc.make_uniform_index(B, H, S // 128, S // 128, count, gen).cuda()
    out, lse = bsa_attn_fwd(q, k, v, index, count, return_lse=True, sparse_block_size=128)
    dq, dk, dv = bsa_attn_bwd(do, q, k, v, out, lse, index, count, sparse_block_size=128)
    full = {"out": out, "lse": lse, "dq": dq, "dk": dk, "dv": dv}
    for world in (1, 2, 4):
        seen = []
        for rank in range(world):
            mine = shard_batch_heads(B, H, world, rank)
            seen += mine
            if not mine:
                continue
            res = sharded_fwd_bwd(q, k, v, do, index, count, mine)
            for i, (b, h) in enumerate(mine):
                for name, t in full.items():
                    assert torch.equal(res[name][0, i], t[b, h]), (world, rank, name, b, h)
        assert sorted(seen) == [(b, h) for b in range(B) for h in range(H)]
