"""Shared helpers of the test-suite (loading golden vectors, tolerances)."""
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def bf16_roundtrip_eps(ref: torch.Tensor) -> float:
    """max |(x + 0.3 - 0.3) - x|: the absolute slack term of the reference's tolerance formula
    (tests/test_flash_fwd.py:322-323)."""
    return (ref + 0.3 - 0.3 - ref).abs().max().item()
