"""Shared helpers for the tests: seeded inputs and torch <-> numpy bit views."""
import numpy as np
import torch


def randn_bf16(shape, seed, std=1.0, outlier_frac=0.0, outlier_scale=32.0):
    """bf16 ~ N(0, std) from a seeded CPU generator; optionally a fraction of entries scaled up."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g, dtype=torch.float32) * std
    if outlier_frac > 0:
        mask = torch.rand(*shape, generator=g) < outlier_frac
        x = torch.where(mask, x * outlier_scale, x)
    return x.to(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def bits_to_bf16(a: np.ndarray, device=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a, np.uint16)).view(torch.bfloat16)
    return t.to(device) if device is not None else t


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def to_dev_u8(a: np.ndarray, device, dtype=torch.uint8) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, np.uint8)).to(device).view(dtype)


def rel_fro(d: np.ndarray, ref: np.ndarray) -> float:
    d = d.astype(np.float64)
    ref = ref.astype(np.float64)
    return float(np.linalg.norm(d - ref) / max(np.linalg.norm(ref), 1e-300))


def bf16_ulp_diff(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in bf16 units-in-the-last-place between two bf16 bit arrays (sign-magnitude aware)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7fff), x & 0x7fff)
    return np.abs(key(a_bits) - key(b_bits))
