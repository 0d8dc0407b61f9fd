"""GPU: a bounded device-side wait that runs out.  A one-CTA kernel waits 2 ms on an mbarrier nobody arrives
at, through the same wait routine the attention kernels use; the kernel must return by itself, leave the
status word {1, block, site, thread}, make check_device_status() raise, and leave the device usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_expires_reports_and_returns():
    from block_sparse_attention import _cabi, bsa_attn_fwd, check_device_status
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    check_device_status(dev)  # clean slate
    status = _cabi.status_buffer(dev)
    returned = torch.zeros(1, dtype=torch.int32, device=dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    _cabi.check(lib.bsa_selftest_wait(2_000_000, status.data_ptr(), returned.data_ptr(), _cabi.stream_ptr(dev)),
                "bsa_selftest_wait")
    t1.record()
    torch.cuda.synchronize()
    assert 1.5 <= t0.elapsed_time(t1) < 500.0  # the wait really ran for its budget, and only for it
    assert returned.item() == 1  # the kernel left through the common exit with the abort answer
    code, block, site, thread = status.tolist()
    assert code == 1 and block == 0 and site in (900, 901) and 0 <= thread < 64
    with pytest.raises(RuntimeError, match="bounded wait expired"):
        check_device_status(dev)
    check_device_status(dev)  # the report was consumed
    # the context is intact: a forward right after works and reports nothing
    q = torch.randn(1, 1, 128, 128, device=dev).bfloat16()
    idx = torch.zeros(1, 1, 1, 1, dtype=torch.int32, device=dev)
    out, _ = bsa_attn_fwd(q, q, q, idx, 1, sparse_block_size=128)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    check_device_status(dev)


def test_selftest_rejects_bad_arguments():
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    buf = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert lib.bsa_selftest_wait(0, buf.data_ptr(), buf.data_ptr(), None) < 0
    assert lib.bsa_selftest_wait(2_000_000_000, buf.data_ptr(), buf.data_ptr(), None) < 0
    assert lib.bsa_selftest_wait(1000, None, buf.data_ptr(), None) < 0
