"""Shared test helpers: torch <-> numpy views of BF16 bits, device upload of oracle-side weights, tolerances."""
import numpy as np
import torch

from strixite_b200.kernels import QDeviceView


def bits_of(t: torch.Tensor) -> np.ndarray:
    """A BF16 (or int16 bit) tensor as numpy uint16."""
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return t.detach().cpu().numpy().view(np.uint16)


def bf16_tensor(bits: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(torch.bfloat16)


def upload(w, device) -> QDeviceView:
    """An oracle-side QWeight onto the device."""
    q = torch.from_numpy(np.ascontiguousarray(w.q)).to(device)
    s = torch.from_numpy(np.ascontiguousarray(w.scale).view(np.int16)).to(device)
    m = torch.from_numpy(np.ascontiguousarray(w.minv).view(np.int16)).to(device)
    return QDeviceView(q, s, m, w.N, w.K, w.G, w.bits)


def download(v: QDeviceView, cpu_mod):
    return cpu_mod.QWeight(v.q.cpu().numpy(), v.scale.cpu().numpy().view(np.uint16),
                           v.minv.cpu().numpy().view(np.uint16), v.N, v.K, v.G, v.bits)


def rms(a: np.ndarray) -> float:
    return float(np.sqrt(np.mean(np.square(a.astype(np.float64)))))


def max_abs_over_rms(got: np.ndarray, ref: np.ndarray) -> float:
    """The acceptance metric of the layer outputs: max |got - ref| / rms(ref); the bar is 1e-2."""
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / max(rms(ref), 1e-30)


def bf16_ulps(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in BF16 units of last place between two arrays of BF16 bits (finite values)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - (u & 0x7FFF), 0x8000 + (u & 0x7FFF))
    return np.abs(key(a_bits) - key(b_bits))


def random_weights(rng, n, k, std=0.02):
    return (rng.standard_normal((n, k)) * std).astype(np.float32)
