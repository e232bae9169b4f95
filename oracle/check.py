"""Checker-side helpers shared by the tests, the smoke check and the benchmark's parity / CPU-baseline legs:
torch <-> numpy views of BF16 bits, download of device-side weights for the oracle, the acceptance metric, and the
oracle run on a subset of a large layer's rows.

TEST INFRASTRUCTURE: nothing in the shipped package imports this module.
"""
from __future__ import annotations

import numpy as np

from . import cpu


def bits_of(t) -> np.ndarray:
    """A BF16 (or int16 bit) tensor as numpy uint16."""
    import torch
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return t.detach().cpu().numpy().view(np.uint16)


def download(v, cpu_mod=cpu):
    """A device-side quantized view (strixite_b200.kernels.QDeviceView) as an oracle-side QWeight."""
    return cpu_mod.QWeight(v.q.cpu().numpy(), v.scale.cpu().numpy().view(np.uint16),
                           v.minv.cpu().numpy().view(np.uint16), v.N, v.K, v.G, v.bits)


def rms(a: np.ndarray) -> float:
    return float(np.sqrt(np.mean(np.square(a.astype(np.float64)))))


def max_abs_over_rms(got: np.ndarray, ref: np.ndarray) -> float:
    """The acceptance metric of the layer outputs: max |got - ref| / rms(ref); the bar is 1e-2."""
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / max(rms(ref), 1e-30)


def take_experts(view, rows_per_expert: int, experts: np.ndarray, cpu_mod=cpu):
    """The stacked rows of `experts` (ascending ids) of a device-side view, as one oracle-side QWeight."""
    import torch
    idx = torch.from_numpy(np.concatenate([np.arange(e * rows_per_expert, (e + 1) * rows_per_expert) for e in experts]))
    idx = idx.to(view.q.device)
    return cpu_mod.QWeight(view.q[idx].cpu().numpy(), view.scale[idx].cpu().numpy().view(np.uint16),
                           view.minv[idx].cpu().numpy().view(np.uint16), len(experts) * rows_per_expert, view.K, view.G,
                           view.bits)


def oracle_layer_with(oracle, cfg, fetch, shared, x_bits, logits, semantics, threads=0):
    """The oracle on a handful of token rows of a large layer.  x_bits [n, d], logits [n, E + 1] (those rows').
    fetch(which, experts) -> QWeight of the stacked rows of `experts` (ascending ids), which = "gate_up" | "down";
    shared: None or (QWeight gate_up, QWeight down).  Only the experts the rows are routed to are fetched."""
    ids, _ = oracle.moe_router(logits, cfg.E, cfg.k)
    touched = np.unique(ids)
    lw = oracle.LayerWeights(fetch("gate_up", touched), fetch("down", touched))
    if shared is not None:
        lw.shared_gate_up, lw.shared_down = shared
    # the oracle routes on the original logits; present it logits whose columns are the touched experts only
    E2 = len(touched)
    sub = np.full((logits.shape[0], E2 + 1), -1e30, dtype=np.float32)
    sub[:, :E2] = logits[:, touched]
    sub[:, E2] = logits[:, cfg.E]
    out = oracle.moe_layer(x_bits, sub, lw, E2, cfg.k, semantics=semantics, threads=threads)
    assert np.array_equal(touched[out["ids"]], ids)  # same picks through the remapping
    out["ids"] = ids
    return out


def oracle_layer_on_touched_experts(oracle, cfg, w, x_bits, logits, rows, semantics, threads=0, e_lo=0):
    """Runs the oracle on the token subset `rows`, downloading only the experts those tokens are routed to (the stacked
    matrices of the large configurations are gigabytes; rows are independent).  `w` holds experts [e_lo, e_lo + n) of
    the layer on the device; every expert the rows pick must be among them."""
    def fetch(which, experts):
        view, n = (w.gate_up, 2 * cfg.I) if which == "gate_up" else (w.down, cfg.d)
        return take_experts(view, n, experts - e_lo, oracle)
    shared = None
    if getattr(w, "shared_gate_up", None) is not None:
        shared = (download(w.shared_gate_up, oracle), download(w.shared_down, oracle))
    return oracle_layer_with(oracle, cfg, fetch, shared, x_bits[rows], logits[rows], semantics, threads)


def generated_experts(cfg, seed, layer, device, order=None):
    """fetch() for oracle_layer_with that REGENERATES the asked experts of a synthetic layer instead of downloading them
    (strixite_b200.workloads draws every expert from its own seeded generator): any rank can check rows routed to experts
    it does not hold.  Quantized on the device when there is one (bit-identical to the reference's quantizer), else by the
    oracle's quantizer on the host.  order: the experts' placement (position p holds expert order[p]; the ids asked for
    are positions)."""
    import torch
    from strixite_b200 import workloads as W

    def fetch(which, experts):
        bits = cfg.gu_bits if which == "gate_up" else cfg.dn_bits
        G = cfg.group(bits)
        parts = []
        for e in experts:
            w32 = W.expert_weight_f32(cfg, seed, device, which, int(e) if order is None else int(order[int(e)]), layer)
            if torch.device(device).type == "cuda":
                from strixite_b200 import kernels as K
                parts.append(download(K.quantize(w32, G, bits), cpu))
            else:
                parts.append(cpu.quantize(w32.numpy(), G, bits))
        return cpu.QWeight(np.concatenate([p.q for p in parts]), np.concatenate([p.scale for p in parts]),
                           np.concatenate([p.minv for p in parts]), sum(p.N for p in parts), parts[0].K, G, bits)
    return fetch
