"""ctypes binding of libbsa_b200.so (the C ABI declared in include/bsa_b200.h).

The library is the only compute path: when it is missing or cannot be loaded every operator raises
``RuntimeError``; there is no fallback of any kind.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# BSA_B200_LIB points at another build of the same library (e.g. one compiled with development timers)
LIB_PATH = os.environ.get("BSA_B200_LIB") or os.path.join(_HERE, "libbsa_b200.so")

BSA_DTYPE_BF16 = 0
BSA_DTYPE_E4M3 = 1
BSA_DTYPE_F16 = 2

_c_i64x3 = ctypes.c_int64 * 3


class FwdArgs(ctypes.Structure):
    """Mirror of ``struct bsa_fwd_args``."""

    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("q2k_index", ctypes.c_void_p),
        ("q2k_nums", ctypes.c_void_p),
        ("block_sizes", ctypes.c_void_p),
        ("q_scale", ctypes.c_void_p),
        ("k_scale", ctypes.c_void_p),
        ("v_scale", ctypes.c_void_p),
        ("partial_o", ctypes.c_void_p),
        ("partial_lse", ctypes.c_void_p),
        ("work_order", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("q_stride", _c_i64x3),
        ("k_stride", _c_i64x3),
        ("v_stride", _c_i64x3),
        ("o_stride", _c_i64x3),
        ("bs_stride_b", ctypes.c_int64),
        ("bs_stride_h", ctypes.c_int64),
        ("dtype", ctypes.c_int32),
        ("blk", ctypes.c_int32),
        ("B", ctypes.c_int32),
        ("Hq", ctypes.c_int32),
        ("Hkv", ctypes.c_int32),
        ("Sq", ctypes.c_int32),
        ("Sk", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("cap", ctypes.c_int32),
        ("block_sparse_num", ctypes.c_int32),
        ("pack_gqa", ctypes.c_int32),
        ("splits", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("reserved", ctypes.c_int32),
    ]


class BwdArgs(ctypes.Structure):
    """Mirror of ``struct bsa_bwd_args``."""

    _fields_ = [
        ("dout", ctypes.c_void_p),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("q2k_index", ctypes.c_void_p),
        ("q2k_nums", ctypes.c_void_p),
        ("csr_offsets", ctypes.c_void_p),
        ("csr_indices", ctypes.c_void_p),
        ("block_sizes", ctypes.c_void_p),
        ("work_order_q", ctypes.c_void_p),
        ("work_order_kv", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_int64),
        ("do_stride", _c_i64x3),
        ("q_stride", _c_i64x3),
        ("k_stride", _c_i64x3),
        ("v_stride", _c_i64x3),
        ("o_stride", _c_i64x3),
        ("dq_stride", _c_i64x3),
        ("dk_stride", _c_i64x3),
        ("dv_stride", _c_i64x3),
        ("bs_stride_b", ctypes.c_int64),
        ("bs_stride_h", ctypes.c_int64),
        ("blk", ctypes.c_int32),
        ("B", ctypes.c_int32),
        ("H", ctypes.c_int32),
        ("Sq", ctypes.c_int32),
        ("Sk", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("cap", ctypes.c_int32),
        ("block_sparse_num", ctypes.c_int32),
        ("num_q_groups", ctypes.c_int32),
        ("bucket_size_blocks", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("stages", ctypes.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/bsa_b200.h declares
_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
SIGNATURES = {
    "bsa_abi_version": (ctypes.c_int, []),
    "bsa_last_error": (ctypes.c_char_p, []),
    "bsa_num_sms": (ctypes.c_int, [ctypes.c_int]),
    "bsa_selftest_wait": (ctypes.c_int, [ctypes.c_uint64, _vp, _vp, _vp]),
    "bsa_fwd": (ctypes.c_int, [ctypes.POINTER(FwdArgs), _vp]),
    "bsa_fwd_combine": (ctypes.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32,
                                       ctypes.POINTER(ctypes.c_int64), _vp]),
    "bsa_quantize_sage": (ctypes.c_int, [_vp] * 11 + [_i32] * 4 + [_vp]),
    "bsa_quantize_sage_scratch_floats": (ctypes.c_int64, [_i32, _i32, _i32]),
    "bsa_quantize_sage_static": (ctypes.c_int, [_vp] * 9 + [_i32] * 4 + [_vp]),
    "bsa_mask_to_q2k": (ctypes.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]),
    "bsa_q2k_to_k2q": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bsa_lpt_order": (ctypes.c_int, [_vp, _i32, _i32, _vp, _vp, _vp]),
    "bsa_lpt_order_scratch_ints": (ctypes.c_int64, [_i32, _i32]),
    "bsa_build_k2q_csr": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bsa_block_mean": (ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_int64), _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bsa_pooled_scores": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_float, _vp, _vp]),
    "bsa_topk_q2k": (ctypes.c_int, [_vp, ctypes.c_int64, _i32, _i32, _i32, _vp, _vp]),
    "bsa_bwd": (ctypes.c_int, [ctypes.POINTER(BwdArgs), _vp]),
    "bsa_bwd_workspace_bytes": (ctypes.c_int64, [_i32, _i32, _i32, _i32, _i32]),
}

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises RuntimeError when it is absent (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python block-sparse-attention_b200/build.py` "
                "(nvcc, sm_100a). The engine has no other compute path."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        if lib.bsa_abi_version() != 1:
            raise RuntimeError("libbsa_b200.so ABI version mismatch")
        _lib = lib
        return lib


def last_error() -> str:
    return load().bsa_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Maps a negative C return code to the exception type the reference raises for that failure."""
    if rc == 0:
        return
    msg = f"{what}: {last_error()} (code {rc})"
    if rc in (-1, -2):
        raise AssertionError(msg)
    raise RuntimeError(msg)


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def strides3(t: torch.Tensor):
    """(batch, head, seq) element strides of a BHSD view."""
    return _c_i64x3(t.stride(0), t.stride(1), t.stride(2))


_status: Dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] word the kernels write when a bounded wait expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = buf
    return buf


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronises and raises RuntimeError when any kernel reported a device-side failure."""
    items = list(_status.items()) if device is None else [
        (device.index if device.index is not None else torch.cuda.current_device(), status_buffer(device))]
    for idx, buf in items:
        vals = buf.cpu().tolist()
        if vals[0] != 0:
            buf.zero_()
            raise RuntimeError(
                f"bsa kernel on cuda:{idx} reported status {vals[0]} (block {vals[1]}, site {vals[2]}, "
                f"thread {vals[3]}): a bounded wait expired; results of that launch are invalid")
