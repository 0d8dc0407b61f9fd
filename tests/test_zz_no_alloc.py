"""GPU: the scratch-owning quantiser entry point (bsa_quantize_sage_static) against the regular one.

Hosts that cannot hand scratch memory to the library - a server with a frozen memory pool, a C service
without a device allocator - call this variant; it must give exactly what bsa_quantize_sage gives with
caller-provided scratch.  Called twice in a row through the C ABI (the built-in array keeps the previous
call's contents), with a different problem in between, and compared bit for bit.  This file sorts last on
purpose, so a run that stops at the first failure has already been through every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(B, H, Sq, Sk):
    dev = "cuda"
    return dict(
        q8=torch.empty(B, H, Sq, 128, dtype=torch.uint8, device=dev),
        k8=torch.empty(B, H, Sk, 128, dtype=torch.uint8, device=dev),
        v8=torch.empty(B, H, Sk, 128, dtype=torch.uint8, device=dev),
        qs=torch.empty(B, H, Sq, dtype=torch.float32, device=dev),
        ks=torch.empty(B, H, (Sk + 15) // 16, dtype=torch.float32, device=dev),
        vs=torch.empty(H, 128, dtype=torch.float32, device=dev),
    )


def _static(lib, q, k, v):
    B, H, Sq, _ = q.shape
    Sk = k.shape[2]
    o = _buffers(B, H, Sq, Sk)
    rc = lib.bsa_quantize_sage_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o["q8"].data_ptr(),
                                      o["k8"].data_ptr(), o["v8"].data_ptr(), o["qs"].data_ptr(),
                                      o["ks"].data_ptr(), o["vs"].data_ptr(), B, H, Sq, Sk,
                                      torch.cuda.current_stream().cuda_stream)
    return rc, o


def _regular(lib, q, k, v):
    B, H, Sq, _ = q.shape
    Sk = k.shape[2]
    o = _buffers(B, H, Sq, Sk)
    k_mean = torch.empty(B, H, 128, dtype=torch.float32, device="cuda")
    partials = torch.empty(int(lib.bsa_quantize_sage_scratch_floats(B, H, Sk)), dtype=torch.float32, device="cuda")
    rc = lib.bsa_quantize_sage(q.data_ptr(), k.data_ptr(), v.data_ptr(), o["q8"].data_ptr(), o["k8"].data_ptr(),
                               o["v8"].data_ptr(), o["qs"].data_ptr(), o["ks"].data_ptr(), o["vs"].data_ptr(),
                               k_mean.data_ptr(), partials.data_ptr(), B, H, Sq, Sk,
                               torch.cuda.current_stream().cuda_stream)
    return rc, o


def test_static_scratch_quantiser_matches_regular_entry_point_twice():
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    gen = torch.Generator().manual_seed(123)
    cases = []
    for B, H, Sq, Sk in [(2, 3, 300, 2100), (1, 2, 77, 130), (2, 3, 300, 2100)]:
        q = torch.randn(B, H, Sq, 128, generator=gen).bfloat16().cuda()
        k = (torch.randn(B, H, Sk, 128, generator=gen) + 1.5).bfloat16().cuda()
        v = torch.randn(B, H, Sk, 128, generator=gen).bfloat16().cuda()
        cases.append((q, k, v))
    for q, k, v in cases:  # back-to-back calls share the built-in scratch
        rc_s, got = _static(lib, q, k, v)
        rc_r, ref = _regular(lib, q, k, v)
        assert rc_s == 0 and rc_r == 0, _cabi.last_error()
        torch.cuda.synchronize()
        for name in ref:
            assert torch.equal(got[name], ref[name]), name  # same kernels, same inputs: bit-identical


def test_static_scratch_quantiser_rejects_oversized_problems():
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    cap = 1 << 20  # BSA_QUANTIZE_STATIC_SCRATCH_FLOATS in include/bsa_b200.h
    B, H, Sk = 8, 64, 32768  # 8*64*(1+2*32)*128 floats = 4.26 Mi > 1 Mi
    assert B * H * (1 + 2 * ((Sk + 1023) // 1024)) * 128 > cap
    dummy = torch.zeros(16, device="cuda")
    p = dummy.data_ptr()
    rc = lib.bsa_quantize_sage_static(p, p, p, p, p, p, p, p, p, B, H, 128, Sk, torch.cuda.current_stream().cuda_stream)
    assert rc == -4  # BSA_ERR_WORKSPACE: nothing was launched
    assert "exceed the built-in scratch" in _cabi.last_error()


def test_static_scratch_quantiser_at_the_limit():
    """The largest problem the built-in scratch takes, and the first one it does not.  With Sk <= 1024 a call
    needs 3 * B * H * 128 floats (a mean row and two statistics rows per (batch, head)), so 2730 heads fit
    (1 048 320 of 1 048 576 floats) and 2731 do not (1 048 704); the limit cannot be met exactly because
    1 + 2 * ceil(Sk / 1024) is odd."""
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    cap = 1 << 20
    gen = torch.Generator().manual_seed(5)
    H, S = 2730, 16
    assert 3 * H * 128 <= cap < 3 * (H + 1) * 128
    q = torch.randn(1, H + 1, S, 128, generator=gen).bfloat16().cuda()
    k = (torch.randn(1, H + 1, S, 128, generator=gen) + 0.5).bfloat16().cuda()
    v = torch.randn(1, H + 1, S, 128, generator=gen).bfloat16().cuda()
    fit = tuple(t[:, :H].contiguous() for t in (q, k, v))
    rc_s, got = _static(lib, *fit)
    rc_r, ref = _regular(lib, *fit)
    assert rc_s == 0 and rc_r == 0, _cabi.last_error()
    torch.cuda.synchronize()
    for name in ref:
        assert torch.equal(got[name], ref[name]), name
    rc, _ = _static(lib, q, k, v)
    assert rc == -4 and "exceed the built-in scratch" in _cabi.last_error()
