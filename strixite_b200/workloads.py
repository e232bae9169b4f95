"""Seeded synthetic inputs for the five benchmark configurations (no public dataset is involved: shapes and value
distributions only).  C0..C4 in the order of the configuration list:

    C0  T=4,  d=1024, E=64,  top-4,  I=256,  all Q8 G64, no shared expert          (CPU-sized)
    C1  T=16 (2 conversations x 8 rows), d=4096, E=512, top-10, I=1024, Q4 G128 experts + Q8 G64 shared expert
    C2  8 conversations x U[1,8] rows (T <= 64), C1's layer, Q4 gate/up + Q8 down, expert bias N(0, 0.5)
    C3  T=4096, C1's layer
    C4  8 layers, T=16384, Q4 gate/up + Q8 down, Zipf(1.1) expert bias, no shared expert, experts sharded over ranks

x ~ N(0, 1) BF16; router weight ~ N(0, 0.02) FP32 [E + 1, d] (row E = the shared gate); expert weights ~ N(0, 0.02)
FP32, quantized with the Q4 (G = 128) / Q8 (G = 64) quantizers.  Every tensor has its own generator seeded from
(seed, name), so a tensor does not depend on which others were drawn or on which device drew them... except that CPU
and CUDA generators give different streams: a configuration is drawn on one device and copied where it is needed.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, replace
from typing import Optional

import torch


@dataclass(frozen=True)
class MoeConfig:
    name: str
    T: int
    d: int
    E: int
    k: int
    I: int
    gu_bits: int = 4
    dn_bits: int = 4
    shared: bool = True
    layers: int = 1
    bias: str = "none"       # "none" | "normal" (std 0.5) | "zipf" (-1.1 ln rank)
    runs: Optional[tuple] = None  # conversation lengths (ragged batch), informational

    def group(self, bits: int) -> int:
        return 128 if bits == 4 else 64


C0 = MoeConfig("c0_cpu_q8", T=4, d=1024, E=64, k=4, I=256, gu_bits=8, dn_bits=8, shared=False)
C1 = MoeConfig("c1_decode", T=16, d=4096, E=512, k=10, I=1024, runs=(8, 8))
C2 = MoeConfig("c2_ragged", T=64, d=4096, E=512, k=10, I=1024, gu_bits=4, dn_bits=8, bias="normal")
C3 = MoeConfig("c3_prefill", T=4096, d=4096, E=512, k=10, I=1024)
C4 = MoeConfig("c4_ep_stack", T=16384, d=4096, E=512, k=10, I=1024, gu_bits=4, dn_bits=8, shared=False, layers=8,
               bias="zipf")
CONFIGS = {c.name.split("_")[0]: c for c in (C0, C1, C2, C3, C4)}


def gen(seed: int, name: str, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFF)
    return g


def ragged_runs(seed: int, n_runs: int = 8, max_len: int = 8) -> tuple:
    """C2: every conversation's row count, uniform in [1, max_len]."""
    g = gen(seed, "runs", "cpu")
    return tuple(int(v) for v in (1 + torch.floor(torch.rand(n_runs, generator=g) * max_len)).tolist())


def c2_config(seed: int = 0) -> MoeConfig:
    runs = ragged_runs(seed)
    return replace(C2, T=sum(runs), runs=runs)


def activations(cfg: MoeConfig, seed: int, device, T: Optional[int] = None) -> torch.Tensor:
    return torch.randn((T or cfg.T, cfg.d), generator=gen(seed, "x", device), device=device).to(torch.bfloat16)


def router_weight(cfg: MoeConfig, seed: int, device, layer: int = 0) -> torch.Tensor:
    return torch.randn((cfg.E + 1, cfg.d), generator=gen(seed, f"router{layer}", device), device=device) * 0.02


def expert_bias(cfg: MoeConfig, seed: int, device, layer: int = 0) -> torch.Tensor:
    """Per-expert logit bias [E + 1] (0 for the shared gate)."""
    b = torch.zeros(cfg.E + 1, device=device)
    if cfg.bias == "normal":
        b[: cfg.E] = (torch.randn(cfg.E, generator=gen(seed, f"bias{layer}", "cpu")) * 0.5).to(device)
    elif cfg.bias == "zipf":
        rank = torch.randperm(cfg.E, generator=gen(seed, f"bias{layer}", "cpu")).to(torch.float32) + 1.0
        b[: cfg.E] = (-1.1 * torch.log(rank)).to(device)
    return b


def router_logits(x: torch.Tensor, wr: torch.Tensor, bias: torch.Tensor, tf32: bool = False) -> torch.Tensor:
    """FP32 logits [T, E + 1] = x Wr^T + bias (the router projection, upstream of the MoE path).  By default an FP32
    GEMM; tf32 = True lets cuBLAS use TF32 tensor cores (the benchmark's choice for prefill-sized T: the router then
    ranks those logits, whatever produced them)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = bool(tf32)
    try:
        return (x.to(torch.float32) @ wr.t() + bias).contiguous()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def expert_weight_f32(cfg: MoeConfig, seed: int, device, which: str, expert: int, layer: int = 0) -> torch.Tensor:
    """One expert's FP32 matrix: which = "gate_up" [2I, d] | "down" [d, I] | "shared_gate_up" | "shared_down"."""
    shape = (2 * cfg.I, cfg.d) if which.endswith("gate_up") else (cfg.d, cfg.I)
    return torch.randn(shape, generator=gen(seed, f"{which}.{layer}.{expert}", device), device=device) * 0.02


def expert_placement(cfg: MoeConfig, seed: int, device, layer: int, world: int, mode: str = "balanced", calib_tokens: int = 4096):
    """Which expert sits where in an expert-parallel run: a list `order` of the E expert ids, rank r holding the experts
    order[r E / world : (r + 1) E / world] (every rank the same number).  Relabelling experts this way changes nothing
    in the model: the router weight's rows and the experts move together.
      "contiguous": expert e at position e.
      "balanced":   by observed load, as a serving engine places experts from its routing statistics: a calibration batch
                    (other activations than the measured ones: seed + 1000) is routed once, an expert's cost is the
                    128-token tiles it fills, and experts are dealt, heaviest first, to the least loaded rank that still
                    has room.  With a Zipf-skewed router the contiguous split leaves one rank 1.5-1.9x the mean load."""
    if world == 1 or mode == "contiguous":
        return list(range(cfg.E))
    x = activations(cfg, seed + 1000, device, T=calib_tokens).float()
    logits = x @ router_weight(cfg, seed, device, layer).t() + expert_bias(cfg, seed, device, layer)
    ids = logits[:, : cfg.E].topk(cfg.k, dim=1).indices.reshape(-1)
    cnt = torch.bincount(ids, minlength=cfg.E).cpu().double() * (cfg.T / calib_tokens)
    cost = torch.ceil(cnt / 128.0) + 1e-3 * cnt
    cap = cfg.E // world
    load, members = [0.0] * world, [[] for _ in range(world)]
    for e in sorted(range(cfg.E), key=lambda i: (-float(cost[i]), i)):
        r = min((r for r in range(world) if len(members[r]) < cap), key=lambda r: (load[r], r))
        members[r].append(e)
        load[r] += float(cost[e])
    return [e for r in range(world) for e in sorted(members[r])]


def placed_router(cfg: MoeConfig, seed: int, device, layer: int, order):
    """Router weight [E + 1, d] and bias [E + 1] with their expert rows in placement order (row E, the shared gate, last)."""
    rows = torch.tensor(list(order) + [cfg.E], device=device)
    return router_weight(cfg, seed, device, layer)[rows].contiguous(), expert_bias(cfg, seed, device, layer)[rows].contiguous()


def make_layer_weights(cfg: MoeConfig, seed: int, device, layer: int = 0, e_lo: int = 0, e_hi: Optional[int] = None, order=None):
    """Draws and quantizes one layer's experts [e_lo, e_hi) on the device (FP32 never leaves it), expert by expert so
    that a rank holding a slice of the experts gets the same bytes as a rank holding them all.  order: the expert at
    position p is expert order[p] (expert_placement); None = in their own order.
    Returns strixite_b200.layer.MoeWeights with the experts stacked along N."""
    from . import kernels as K
    from .layer import MoeWeights

    e_hi = cfg.E if e_hi is None else e_hi
    n = e_hi - e_lo

    def stacked(which: str, rows: int, cols: int, bits: int):
        G = cfg.group(bits)
        q = torch.empty((n * rows, cols // 2 if bits == 4 else cols), dtype=torch.uint8, device=device)
        s = torch.empty((n * rows, cols // G), dtype=torch.int16, device=device)
        m = torch.empty((n * rows, cols // G), dtype=torch.int16, device=device)
        err = torch.zeros(4, dtype=torch.int32, device=device)
        for i, pos in enumerate(range(e_lo, e_hi)):
            e = pos if order is None else order[pos]
            v = K.quantize(expert_weight_f32(cfg, seed, device, which, e, layer), G, bits, err=err)
            q[i * rows:(i + 1) * rows] = v.q
            s[i * rows:(i + 1) * rows] = v.scale
            m[i * rows:(i + 1) * rows] = v.minv
        return K.QDeviceView(q, s, m, n * rows, cols, G, bits)

    w = MoeWeights(stacked("gate_up", 2 * cfg.I, cfg.d, cfg.gu_bits), stacked("down", cfg.d, cfg.I, cfg.dn_bits))
    if cfg.shared:
        G = cfg.group(8)
        w.shared_gate_up = K.quantize(expert_weight_f32(cfg, seed, device, "shared_gate_up", 0, layer), G, 8)
        w.shared_down = K.quantize(expert_weight_f32(cfg, seed, device, "shared_down", 0, layer), G, 8)
    return w
