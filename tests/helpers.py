"""Shared helpers for the test-suite: seeded synthetic inputs and the library import."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "alice-train_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def rng(seed: int) -> np.random.Generator:
    """Counter-based generator so that every run (and the fixture script) sees identical bits."""
    return np.random.Generator(np.random.Philox(seed))


def normal_f32(seed: int, shape, std: float = 1.0) -> np.ndarray:
    return (rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def rel_err(got, ref) -> float:
    """max |got-ref| over max |ref| : the error measure every floating-point parity check uses."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    denom = max(float(np.max(np.abs(ref))) if ref.size else 0.0, 1e-30)
    return float(np.max(np.abs(got - ref))) / denom if ref.size else 0.0


def to_bf16_tensor(orc, a: np.ndarray, device):
    """f32 numpy -> torch.bfloat16 via the ORACLE's round-to-nearest-even (src/mixed_precision.rs:29-39)."""
    import torch
    bits = orc.bf16_round(a)
    return torch.from_numpy(bits.view(np.int16)).to(device).view(torch.bfloat16), orc.bf16_bits_to_f32(bits)
