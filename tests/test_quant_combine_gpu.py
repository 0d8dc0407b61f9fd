"""GPU parity of the Sage quantiser (bit-level rules of tests/test_bsa_fp8_quant.py:34-63) and of the
split-KV combine against the CPU oracle."""
import ctypes

import pytest
import torch

from oracle import bsa_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,H,Sq,Sk,dist", [(1, 2, 256, 256, "normal"), (2, 3, 200, 1100, "normal"),
                                            (2, 2, 77, 333, "scaled"), (1, 1, 1, 1, "normal"),
                                            (1, 2, 64, 2500, "zero_v")])
def test_quantiser_matches_recipe(B, H, Sq, Sk, dist):
    from block_sparse_attention import quantize_sage_bhsd
    gen = torch.Generator().manual_seed(Sq * 7 + Sk)
    q = torch.randn(B, H, Sq, 128, generator=gen).bfloat16()
    k = torch.randn(B, H, Sk, 128, generator=gen).bfloat16()
    v = torch.randn(B, H, Sk, 128, generator=gen).bfloat16()
    if dist == "zero_v":
        v.zero_()
    elif dist == "scaled":
        ch = torch.logspace(-4, 1, 128)[None, None, None, :]
        q = (q.float() * ch).bfloat16()
        k = (k.float() * ch + 2.0).bfloat16()
        v = (v.float() * ch * torch.arange(1, B + 1)[:, None, None, None]).bfloat16()
    q8, k8, v8, qs, ks, vs = quantize_sage_bhsd(q.cuda(), k.cuda(), v.cuda())
    r_q8, r_k8, r_v8, r_qs, r_ks, r_vs = orc.sage_quantize(q, k, v)
    assert q8.dtype == torch.float8_e4m3fn and all(t.is_contiguous() for t in (q8, k8, v8, qs, ks, vs))
    assert torch.equal(qs.cpu(), r_qs) and torch.equal(vs.cpu(), r_vs)  # scales bit-exact
    assert torch.equal(q8.cpu().view(torch.uint8), r_q8.view(torch.uint8))  # Q bytes bit-exact
    dv = v8.cpu().float() != r_v8.float()
    if dv.any():  # only an adjacent bin at a reciprocal-ULP midpoint
        assert dv.float().mean() < 1e-4
        assert ((v8.cpu().float() - r_v8.float()).abs()[dv] <= 32).all()
    assert torch.allclose(ks.cpu(), r_ks, atol=2e-8, rtol=2e-6)
    assert (k8.cpu().float() != r_k8.float()).float().mean().item() < 1e-4
    assert (k8.cpu().float() - r_k8.float()).abs().max() <= 32.0


def test_quantiser_rejections():
    from block_sparse_attention import quantize_sage_bhsd
    x = torch.zeros(1, 2, 64, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        quantize_sage_bhsd(x, x, x)  # CPU tensors
    xc = x.cuda()
    with pytest.raises(TypeError):
        quantize_sage_bhsd(xc.half(), xc.half(), xc.half())
    with pytest.raises(ValueError):
        quantize_sage_bhsd(xc[..., :64], xc[..., :64], xc[..., :64])
    with pytest.raises(ValueError):
        quantize_sage_bhsd(xc.transpose(1, 2), xc, xc)


@pytest.mark.parametrize("splits,rows_shape", [(2, (1, 2, 130)), (4, (2, 3, 257)), (7, (1, 1, 64)), (16, (1, 2, 33))])
def test_combine_matches_oracle(splits, rows_shape):
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    B, H, Sq = rows_shape
    gen = torch.Generator().manual_seed(splits)
    po = torch.randn(splits, B, H, Sq, 128, generator=gen)
    pl = torch.randn(splits, B, H, Sq, generator=gen) * 3
    pl[0, :, :, ::5] = float("-inf")  # some empty splits
    pl[:, :, :, 7] = float("-inf")    # a fully empty row
    po[:, :, :, 7] = 123.0
    out = torch.empty(B, H, Sq, 128, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda")
    poc, plc = po.cuda(), pl.cuda()
    ostr = (ctypes.c_int64 * 3)(*out.stride()[:3])
    rc = lib.bsa_fwd_combine(poc.data_ptr(), plc.data_ptr(), out.data_ptr(), lse.data_ptr(), splits, B, H, Sq, 128,
                             ostr, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    ref_out, ref_lse = orc.combine_partials(po, pl)
    assert torch.allclose(out.float().cpu(), ref_out, atol=2e-2, rtol=1e-2)
    assert torch.equal(torch.isinf(lse.cpu()), torch.isinf(ref_lse))
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse.cpu()[fin], ref_lse[fin], atol=1e-4)
    assert (out[:, :, 7] == 0).all()
