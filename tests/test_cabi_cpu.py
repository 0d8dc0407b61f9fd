"""CPU: the shared library loads, exports every symbol include/bsa_b200.h declares, and the host mirror
rejects bad arguments before anything touches a GPU."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "bsa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__
    __graft_entry__.build()
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    names = _declared_symbols()
    assert "bsa_fwd" in names and "bsa_bwd" in names and len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n
        assert n in _cabi.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.bsa_abi_version() == 1
    assert lib.bsa_bwd_workspace_bytes(2, 32, 32768, 32768, 128) == 2 * 2 * 32 * 32768 * 4
    assert lib.bsa_quantize_sage_scratch_floats(1, 24, 76800) == 2 * 24 * 75 * 128


def test_struct_layouts_match_header_order():
    from block_sparse_attention import _cabi
    text = open(os.path.join(ROOT, "include", "bsa_b200.h")).read()
    for struct, cls in (("bsa_fwd_args", _cabi.FwdArgs), ("bsa_bwd_args", _cabi.BwdArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.split(None, 1)[1] if decl.startswith("const") else decl
            names = re.sub(r"^(const\s+)?[A-Za-z0-9_]+\s*\**", "", decl).strip()
            names = re.sub(r"^[A-Za-z0-9_]+\s*\*?\s*(?=[A-Za-z_])", "", names) if names.startswith("void") else names
            for n in names.split(","):
                fields.append(re.sub(r"[\*\s]|\[.*\]", "", n))
        assert [f for f in fields if f] == [f[0] for f in cls._fields_], struct


def test_cpu_tensors_and_bad_arguments_raise_assertion_errors():
    from block_sparse_attention import bsa_attn_bwd, bsa_attn_fwd, bsa_fp8_blk128_fwd, bsa_fp8_fwd
    q = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16)
    idx = torch.zeros(1, 2, 1, 2, dtype=torch.int32)
    with pytest.raises(AssertionError):
        bsa_attn_fwd(q, q, q, idx, 2, sparse_block_size=128)  # CPU tensors
    with pytest.raises(AssertionError):
        bsa_attn_fwd(q, q, q, idx, 2, sparse_block_size=100)
    with pytest.raises(AssertionError):
        bsa_attn_fwd(q, q, q, idx, 2, sparse_block_size=64, kv_splits="many")
    with pytest.raises(AssertionError):
        bsa_attn_bwd(q, q, q, q, q, torch.zeros(1, 2, 128), idx, 2, layout="sbhd", sparse_block_size=128)
    q8 = q.to(torch.float8_e4m3fn)
    s = torch.ones(256)
    with pytest.raises(AssertionError):
        bsa_fp8_blk128_fwd(q8, q8, q8, s, s, s, idx, 2, kv_splits=True)   # bool is not an int here
    with pytest.raises(AssertionError):
        bsa_fp8_blk128_fwd(q8, q8, q8, s, s, s, idx, 2, kv_splits=2.0)
    with pytest.raises(AssertionError):
        bsa_fp8_blk128_fwd(q8, q8, q8, s, s, s, idx, 2, kv_splits=257)
    with pytest.raises(AssertionError):
        bsa_fp8_fwd(q8, q8, q8, s, s, s, idx, 2, sparse_block_size=64, kv_splits=2)


def test_c_entry_points_reject_misaligned_pointers_before_any_launch():
    """The kernels use 16-byte vector accesses on several tensors: a C caller passing an unaligned pointer
    gets BSA_ERR_INVALID from the argument check (no CUDA call has been made by then, so this runs without a GPU)."""
    from block_sparse_attention import _cabi
    lib = _cabi.load()
    good, bad = 0x10000, 0x10008
    a = _cabi.BwdArgs()
    for name in ("dout", "q", "k", "v", "out", "lse", "dq", "dk", "dv", "q2k_index", "csr_offsets", "csr_indices",
                 "workspace", "status"):
        setattr(a, name, good)
    a.blk, a.B, a.H, a.Sq, a.Sk, a.D, a.cap, a.block_sparse_num, a.num_q_groups = 128, 1, 1, 128, 128, 128, 1, 1, 1
    a.workspace_bytes = int(lib.bsa_bwd_workspace_bytes(1, 1, 128, 128, 128))
    for t in ("do_stride", "q_stride", "k_stride", "v_stride", "o_stride", "dq_stride", "dk_stride", "dv_stride"):
        setattr(a, t, _cabi._c_i64x3(128 * 128, 128 * 128, 128))
    for name in ("out", "dout", "dq", "dk", "dv"):
        setattr(a, name, bad)
        assert lib.bsa_bwd(a, None) == -1 and "16-byte aligned" in _cabi.last_error() and name in _cabi.last_error()
        setattr(a, name, good)
    a.stages = 8
    assert lib.bsa_bwd(a, None) == -1 and "stages" in _cabi.last_error()
    # quantiser: q, k, v, q8, k8, v8, k_mean
    args = [good] * 11
    for i in (0, 1, 2, 3, 4, 5, 9):
        args[i] = bad
        assert lib.bsa_quantize_sage(*args, 1, 1, 16, 16, None) == -1 and "16-byte aligned" in _cabi.last_error()
        args[i] = good
    # forward: the output rows are stored as 16-byte vectors
    f = _cabi.FwdArgs()
    for name in ("q", "k", "v", "out", "q2k_index", "status"):
        setattr(f, name, good)
    f.blk, f.B, f.Hq, f.Hkv, f.Sq, f.Sk, f.D, f.cap, f.block_sparse_num, f.splits = 128, 1, 1, 1, 128, 128, 128, 1, 1, 1
    f.softmax_scale = 0.1
    for t in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(f, t, _cabi._c_i64x3(128 * 128, 128 * 128, 128))
    f.out = bad
    assert lib.bsa_fwd(f, None) == -1 and "16-byte aligned" in _cabi.last_error()
    f.out = good
    f.o_stride = _cabi._c_i64x3(128 * 128, 128 * 128, 100)
    assert lib.bsa_fwd(f, None) == -1 and "multiples of 8" in _cabi.last_error()


def test_quantiser_rejections_on_cpu():
    from block_sparse_attention import quantize_sage_bhsd
    x = torch.zeros(1, 2, 64, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        quantize_sage_bhsd(x[0], x[0], x[0])
    with pytest.raises(TypeError):
        quantize_sage_bhsd(x.float(), x.float(), x.float())
    with pytest.raises(ValueError):
        quantize_sage_bhsd(x, x, x)  # not CUDA


def test_policies_and_public_names():
    import block_sparse_attention as bsa
    from block_sparse_attention import bsa_attn_interface as iface
    for name in ("bsa_attn_fwd", "bsa_attn_bwd", "bsa_fp8_fwd", "bsa_fp8_blk64_fwd", "bsa_fp8_blk128_fwd",
                 "quantize_sage_bhsd", "convert_q2k_to_k2q"):
        assert callable(getattr(bsa, name))
    assert [iface._sm100_blk64_kv_splits_from_count(c) for c in (1, 255, 256, 450, 900)] == [1, 1, 2, 4, 8]
    assert iface.sm100_blk128_bwd_default_bucketed_k2q_size_blocks(256, 32) == 384
    assert iface.sm100_blk128_bwd_default_bucketed_k2q_size_blocks(2048, 8) == 512
    assert iface.sm100_blk128_bwd_default_bucketed_k2q_size_blocks(4096, 1) == 256
    import inspect
    sig = inspect.signature(bsa.bsa_fp8_blk128_fwd)
    assert list(sig.parameters) == ["q_fp8", "k_fp8", "v_fp8", "q_sfs", "k_sfs", "v_sfs", "q2k_block_index",
                                    "topk_num", "softmax_scale", "block_sizes", "q2k_block_nums", "kv_splits"]
    sig = inspect.signature(bsa.bsa_attn_fwd)
    assert list(sig.parameters)[:6] == ["q", "k", "v", "q2k_block_index", "block_sparse_num", "block_sizes"]
    assert sig.parameters["sparse_block_size"].default == 64 and sig.parameters["kv_splits"].default == 1


def test_custom_ops_trace_with_fake_tensors_on_cpu():
    """torch.ops.bsa_b200.fwd has a shape-only implementation: a graph can be traced without a GPU."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode
    from block_sparse_attention import block_sparse_attention_op
    with FakeTensorMode():
        q = torch.empty(2, 4, 512, 128, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 4, 768, 128, dtype=torch.bfloat16, device="cuda")
        idx = torch.empty(2, 4, 4, 3, dtype=torch.int32, device="cuda")
        out = block_sparse_attention_op(q, k, k, idx, 3)
        assert out.shape == q.shape and out.dtype == torch.bfloat16
        o2, lse = torch.ops.bsa_b200.fwd(q.transpose(1, 2), k.transpose(1, 2), k.transpose(1, 2), idx, 3, None, None,
                                         0.1, 128, "bshd")
        assert o2.shape == (2, 512, 4, 128) and lse.shape == (2, 4, 512) and lse.dtype == torch.float32
        dq, dk, dv = torch.ops.bsa_b200.bwd(out, q, k, k, out, lse, idx, 3, None, None, 0.1, 128, "bhsd")
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape
