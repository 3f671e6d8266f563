"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import numpy as np


def normwise(got, want) -> float:
    """max|got - want| / max|want| : the error measure the tolerances are stated in."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def bits_to_torch(bits: np.ndarray, dtype, device="cuda"):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(dtype)


def torch_to_bits(t) -> np.ndarray:
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
