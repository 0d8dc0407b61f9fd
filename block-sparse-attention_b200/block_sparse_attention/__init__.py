"""B200-native block-sparse attention: drop-in for the public names of the reference package
(block_sparse_attention/__init__.py:19-63), resolved lazily."""
from __future__ import annotations

import importlib

_EXPORTS = {
    "bsa_attn_fwd": ".bsa_attn_interface",
    "bsa_attn_bwd": ".bsa_attn_interface",
    "bsa_fp8_fwd": ".bsa_attn_interface",
    "bsa_fp8_blk64_fwd": ".bsa_attn_interface",
    "bsa_fp8_blk128_fwd": ".bsa_attn_interface",
    "convert_q2k_to_k2q": ".bsa_attn_interface",
    "block_mask_to_q2k": ".bsa_attn_interface",
    "check_device_status": ".bsa_attn_interface",
    "quantize_sage_bhsd": ".bsa_fp8_quant",
    "block_sparse_attention": ".autograd",
    "HostPipeline": ".host_pipeline",
    "BlockSparseAttentionFunction": ".autograd",
    "block_sparse_attention_op": ".torch_ops",
    "block_mean": ".topk_index",
    "pooled_scores": ".topk_index",
    "topk_q2k": ".topk_index",
    "pooled_topk_q2k": ".topk_index",
}

__all__ = sorted(_EXPORTS)
__version__ = "0.1.0"


def __getattr__(name):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(mod, __name__), name)
    globals()[name] = value
    return value
