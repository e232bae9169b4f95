"""Expert-parallel MoE stack over torch.distributed (one process per GPU; NCCL over NVLink on GPUs, gloo in the CPU
tests of this plumbing).  No counterpart in the reference, which drives one GPU.

Rank r of N owns experts [r * E / N, (r + 1) * E / N) of every layer and the token rows [r * T / N, (r + 1) * T / N).
Per layer:
    1. router logits and top-k on the rank's own rows                      (replicated router weight)
    2. all-gather of the activations [T/N, d] -> [T, d] and of ids | coef  (the exchange into the experts)
    3. pack restricted to the rank's experts, grouped gate/up + SwiGLU, grouped down + combine
       -> this rank's partial sum of every row, zeros where it serves none of a row's experts
    4. reduce-scatter (sum, FP32) of the partial rows -> the rank's own rows (the exchange out of the experts)
    5. residual: x <- bf16(x + y)
With N = 1 steps 2 and 4 vanish and the kernels are exactly the single-GPU layer's.

The compute steps are injected (`Compute`), so the exchange logic can be exercised on CPU ranks with a stand-in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


@dataclass
class Compute:
    """The per-rank device work of one layer.
    route(layer, x_loc [t, d]) -> (ids [t, k] int32, coef [t, k] float32)
    experts(layer, x_all [T, d], ids_all [T, k], coef_all [T, k]) -> y_partial [T, d] float32"""

    route: Callable
    experts: Callable


def shard_bounds(total: int, world: int, rank: int):
    """Contiguous equal shards; `total` must divide evenly (checked by the caller's configuration)."""
    if total % world:
        raise ValueError(f"{total} does not divide over {world} ranks")
    n = total // world
    return rank * n, (rank + 1) * n


class ExpertParallelMoe:
    def __init__(self, compute: Compute, n_layers: int, T: int, d: int, k: int, device, group=None):
        self.c = compute
        self.layers = n_layers
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.T, self.d, self.k = T, d, k
        self.t_lo, self.t_hi = shard_bounds(T, self.world, self.rank)
        t = self.t_hi - self.t_lo
        if self.world > 1:
            self.x_all = torch.empty((T, d), dtype=torch.bfloat16, device=device)
            self.route_loc = torch.empty((t, 2 * k), dtype=torch.int32, device=device)   # ids | coef bits
            self.route_all = torch.empty((T, 2 * k), dtype=torch.int32, device=device)
            self.y_loc = torch.empty((t, d), dtype=torch.float32, device=device)

    def layer(self, l: int, x_loc: torch.Tensor) -> torch.Tensor:
        """One layer on this rank's rows; returns y [t, d] float32 (the full sum over all ranks' experts)."""
        ids, coef = self.c.route(l, x_loc)
        if self.world == 1:
            return self.c.experts(l, x_loc, ids, coef)
        k = self.k
        self.route_loc[:, :k] = ids
        self.route_loc[:, k:] = coef.view(torch.int32)
        dist.all_gather_into_tensor(self.x_all, x_loc.contiguous(), group=self.group)
        dist.all_gather_into_tensor(self.route_all, self.route_loc, group=self.group)
        ids_all = self.route_all[:, :k].contiguous()
        coef_all = self.route_all[:, k:].contiguous().view(torch.float32)
        y_part = self.c.experts(l, self.x_all, ids_all, coef_all)
        dist.reduce_scatter_tensor(self.y_loc, y_part, op=dist.ReduceOp.SUM, group=self.group)
        return self.y_loc

    def forward(self, x_loc: torch.Tensor, keep: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """The stack: x <- bf16(x + moe_l(x)) for every layer; returns this rank's rows after the last layer."""
        x = x_loc
        for l in range(self.layers):
            y = self.layer(l, x)
            if keep is not None:
                keep.append(y.clone())
            x = (x.to(torch.float32) + y).to(torch.bfloat16)
        return x
