"""Helpers shared by the tests: golden-file access and torch <-> oracle conversions."""
from __future__ import annotations

from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name: str):
    return np.load(GOLDEN / f"{name}.npz")


def to_f32(bits: np.ndarray, T: str) -> np.ndarray:
    """Stored raw bits of a T tensor -> float32 values."""
    if T == "f32":
        return np.asarray(bits, dtype=np.float32)
    if T == "f16":
        return bits.view(np.float16).astype(np.float32)
    if T == "bf16":
        return (bits.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(T)


def same_bits(a: np.ndarray, b: np.ndarray) -> bool:
    """float32 arrays equal bit for bit (NaN == NaN, -0 != +0)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    if a.shape != b.shape:
        return False
    an, bn = np.isnan(a), np.isnan(b)
    return bool(np.array_equal(an, bn) and np.array_equal(a.view(np.uint32)[~an], b.view(np.uint32)[~bn]))


def same_values(a: np.ndarray, b: np.ndarray) -> bool:
    """Equal as numbers (NaN == NaN, -0 == +0)."""
    return bool(np.array_equal(np.asarray(a, np.float32), np.asarray(b, np.float32), equal_nan=True))


# ---- torch side (imported lazily so that pure-oracle tests do not need torch) ----------------

def torch_dtype(T: str):
    import torch

    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[T]


def tensor_from_f32(x: np.ndarray, T: str, device="cuda"):
    """float32 values (exactly representable in T) -> torch tensor of dtype T on device."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch_dtype(T)).to(device)


def f32_from_tensor(t) -> np.ndarray:
    return t.detach().float().cpu().numpy()
