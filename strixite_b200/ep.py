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

Micro-batches.  The rows of a MoE layer stack are independent of one another from the first layer to the last, so a rank may
cut its rows into `micro` chunks and run each chunk's whole stack as its own sequence of launches on its own stream: while
one chunk is in its all-gather or reduce-scatter (NVLink, a few SMs), the other chunk's grouped GEMMs have the tensor
cores.  Every chunk needs its own set of work buffers: the compute callbacks get the chunk number.  Within a layer the
all-gather of the activations is started before the routing it does not depend on.

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
    experts(layer, x_all [T, d], ids_all [T, k], coef_all [T, k]) -> y_partial [T, d] float32
    With micro-batches (`chunked = True`) both take the chunk number as a last argument and t, T are a chunk's."""

    route: Callable
    experts: Callable
    chunked: bool = False


def shard_bounds(total: int, world: int, rank: int):
    """Contiguous equal shards; `total` must divide evenly (checked by the caller's configuration)."""
    if total % world:
        raise ValueError(f"{total} does not divide over {world} ranks")
    n = total // world
    return rank * n, (rank + 1) * n


def residual(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """bf16(x + y) with the sum in FP32: one elementwise pass (x BF16, y FP32 in, BF16 out) - the library's kernel on a
    GPU, torch's on the CPU ranks of the plumbing tests."""
    out = torch.empty_like(x)
    if x.is_cuda:
        from . import kernels as K
        K.residual_add(x, y, out)
    else:
        torch.add(x, y, out=out)
    return out


class ExpertParallelMoe:
    def __init__(self, compute: Compute, n_layers: int, T: int, d: int, k: int, device, group=None, micro: int = 1,
                 exchange: str = "reduce_scatter"):
        self.c = compute
        self.layers = n_layers
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.T, self.d, self.k = T, d, k
        self.t_lo, self.t_hi = shard_bounds(T, self.world, self.rank)
        t = self.t_hi - self.t_lo
        self.micro = micro if (self.world > 1 and micro > 1 and compute.chunked and t % micro == 0) else 1
        self.streams = None
        self.exchange = exchange  # how the partial rows come back: "reduce_scatter" (NCCL's) or "a2a" (all-to-all + local sum)
        # set to a list to record CUDA events around the phases of every layer (rank-local; see timing_summary)
        self.timing = None
        if self.world > 1:
            tc, Tc = t // self.micro, T // self.micro
            self.x_all = [torch.empty((Tc, d), dtype=torch.bfloat16, device=device) for _ in range(self.micro)]
            self.route_loc = [torch.empty((tc, 2 * k), dtype=torch.int32, device=device) for _ in range(self.micro)]   # ids | coef bits
            self.route_all = [torch.empty((Tc, 2 * k), dtype=torch.int32, device=device) for _ in range(self.micro)]
            self.y_loc = [torch.empty((tc, d), dtype=torch.float32, device=device) for _ in range(self.micro)]
            if exchange == "a2a":
                self.pieces = [torch.empty((self.world, tc, d), dtype=torch.float32, device=device) for _ in range(self.micro)]

    def _route(self, l, x, chunk):
        return self.c.route(l, x, chunk) if self.c.chunked else self.c.route(l, x)

    def _experts(self, l, x_all, ids, coef, chunk):
        return self.c.experts(l, x_all, ids, coef, chunk) if self.c.chunked else self.c.experts(l, x_all, ids, coef)

    def layer(self, l: int, x_loc: torch.Tensor, chunk: int = 0) -> torch.Tensor:
        """One layer on this rank's rows (of one chunk); returns y [t, d] float32 (the full sum over all ranks' experts)."""
        if self.world == 1:
            ids, coef = self._route(l, x_loc, chunk)
            return self._experts(l, x_loc, ids, coef, chunk)
        k = self.k
        x_all, route_loc, route_all = self.x_all[chunk], self.route_loc[chunk], self.route_all[chunk]
        marks = []

        def mark():
            if self.timing is not None and x_loc.is_cuda:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)
        mark()
        gather_x = dist.all_gather_into_tensor(x_all, x_loc.contiguous(), group=self.group, async_op=True)  # under the routing
        ids, coef = self._route(l, x_loc, chunk)
        route_loc[:, :k] = ids
        route_loc[:, k:] = coef.view(torch.int32)
        mark()  # routing issued
        gather_r = dist.all_gather_into_tensor(route_all, route_loc, group=self.group, async_op=True)
        gather_x.wait()
        gather_r.wait()
        ids_all = route_all[:, :k].contiguous()
        coef_all = route_all[:, k:].contiguous().view(torch.float32)
        mark()  # gathers landed
        y_part = self._experts(l, x_all, ids_all, coef_all, chunk)
        mark()  # experts issued
        if self.exchange == "a2a":
            # every rank sends each peer that peer's rows of its partial sums directly (all links of the switch at once)
            # and adds up the N pieces it receives, in rank order
            pieces = self.pieces[chunk]
            dist.all_to_all_single(pieces.view(-1), y_part.reshape(-1), group=self.group)
            torch.sum(pieces, dim=0, out=self.y_loc[chunk])
        else:
            dist.reduce_scatter_tensor(self.y_loc[chunk], y_part, op=dist.ReduceOp.SUM, group=self.group)
        mark()  # reduce-scatter
        if marks:
            self.timing.append(marks)
        return self.y_loc[chunk]

    def timing_summary(self):
        """Mean milliseconds per layer of (routing, waiting for the gathers, experts, reduce-scatter); needs a device sync."""
        if not self.timing:
            return None
        torch.cuda.synchronize()
        n = len(self.timing)
        names = ("route", "gather_wait", "experts", "reduce_scatter")
        out = {nm: sum(m[i].elapsed_time(m[i + 1]) for m in self.timing) / n for i, nm in enumerate(names)}
        self.timing.clear()
        return out

    def forward(self, x_loc: torch.Tensor, keep: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """The stack: x <- bf16(x + moe_l(x)) for every layer; returns this rank's rows after the last layer."""
        if self.micro == 1:
            x = x_loc
            for l in range(self.layers):
                y = self.layer(l, x)
                if keep is not None:
                    keep.append(y.clone())
                x = residual(x, y)
            return x
        # micro-batches: chunk c's launches go to stream c; layers alternate between the chunks so that one chunk's
        # collectives are in flight while the other's kernels run
        cuda = x_loc.is_cuda
        tc = x_loc.shape[0] // self.micro
        xs = [x_loc[c * tc:(c + 1) * tc] for c in range(self.micro)]
        if cuda:
            if self.streams is None:
                self.streams = [torch.cuda.Stream(device=x_loc.device) for _ in range(self.micro)]
            cur = torch.cuda.current_stream()
            for st in self.streams:
                st.wait_stream(cur)
        for l in range(self.layers):
            for c in range(self.micro):
                if cuda:
                    with torch.cuda.stream(self.streams[c]):
                        y = self.layer(l, xs[c], c)
                        if keep is not None:
                            keep.append(y.clone())  # on the chunk's stream: y is overwritten by its next layer there
                        xs[c] = residual(xs[c], y)
                else:
                    y = self.layer(l, xs[c], c)
                    if keep is not None:
                        keep.append(y.clone())
                    xs[c] = residual(xs[c], y)
        if cuda:
            for st in self.streams:
                cur.wait_stream(st)
            out = torch.cat(xs)
            for t in xs:
                t.record_stream(cur)
            return out
        return torch.cat(xs)
