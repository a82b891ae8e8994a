"""Helpers shared by the parity tests."""
import numpy as np


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    """||a - b|| / ||b|| in float64."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def dev(x):
    """numpy -> CUDA tensor (torch is only the device-memory allocator here)."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()
