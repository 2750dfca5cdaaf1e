"""Shared helpers of the parity tests: seeded synthetic tensors and bf16 <-> numpy bridges."""
from __future__ import annotations

import numpy as np

import oracle_bridge as ob


def bf16_normal(rng: np.random.Generator, shape, std: float = 1.0) -> np.ndarray:
    """bf16 bit patterns (uint16) of N(0, std) samples."""
    return ob.f32_to_bf16((rng.standard_normal(shape) * std).astype(np.float32))


def activations(rng: np.random.Generator, M: int, K: int, outliers: int = 32) -> np.ndarray:
    """bf16 N(0,1) activations with `outliers` fixed channels scaled x16 (benchmark configuration 0)."""
    x = rng.standard_normal((M, K)).astype(np.float32)
    chans = np.random.default_rng(0).choice(K, size=min(outliers, K), replace=False)
    x[:, chans] *= 16.0
    return ob.f32_to_bf16(x)


def to_torch_bf16(bits: np.ndarray, device="cuda"):
    import torch
    return torch.from_numpy(bits.view(np.int16).copy()).to(device).view(torch.bfloat16)


def from_torch_bf16(t) -> np.ndarray:
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rel_l2(c: np.ndarray, r: np.ndarray) -> float:
    c = c.astype(np.float64).ravel()
    r = r.astype(np.float64).ravel()
    return float(np.sqrt(np.sum((c - r) ** 2) / max(np.sum(r ** 2), 1e-300)))


def cosine(c: np.ndarray, r: np.ndarray) -> float:
    c = c.astype(np.float64).ravel()
    r = r.astype(np.float64).ravel()
    return float(np.dot(c, r) / max(np.linalg.norm(c) * np.linalg.norm(r), 1e-300))
