"""Shared test helpers: torch <-> numpy views of BF16 bits, device upload of oracle-side weights, tolerances."""
import numpy as np
import torch

from oracle.check import bits_of, download, max_abs_over_rms, oracle_layer_on_touched_experts, rms  # noqa: F401
from strixite_b200.kernels import QDeviceView


def bf16_tensor(bits: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(torch.bfloat16)


def upload(w, device) -> QDeviceView:
    """An oracle-side QWeight onto the device."""
    q = torch.from_numpy(np.ascontiguousarray(w.q)).to(device)
    s = torch.from_numpy(np.ascontiguousarray(w.scale).view(np.int16)).to(device)
    m = torch.from_numpy(np.ascontiguousarray(w.minv).view(np.int16)).to(device)
    return QDeviceView(q, s, m, w.N, w.K, w.G, w.bits)


def bf16_ulps(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in BF16 units of last place between two arrays of BF16 bits (finite values)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - (u & 0x7FFF), 0x8000 + (u & 0x7FFF))
    return np.abs(key(a_bits) - key(b_bits))


def random_weights(rng, n, k, std=0.02):
    return (rng.standard_normal((n, k)) * std).astype(np.float32)
