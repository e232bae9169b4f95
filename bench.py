#!/usr/bin/env python
"""Benchmark of the quantized MoE FFN path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c3|c2|c1] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

One JSON line on rank 0.  The headline workload (every N) is C4, the configuration the metric "MoE-layer tokens/s at
1/2/4/8 B200" is quoted on: a stack of 8 MoE layers, T = 16384 prefill tokens, hidden 4096, 512 experts (512 / N per
GPU), top-10, intermediate 1024, Q4 G128 gate/up and Q8 G64 down, Zipf(1.1) expert popularity; synthetic seeded inputs
(strixite_b200/workloads.py).  A step = one pass of the T tokens through the 8 layers (router projection, router top-k,
pack, gate/up + SwiGLU, down + combine, residual; with N > 1 an all-gather of activations and a reduce-scatter of expert
outputs per layer).  value = T * layers / step time, "MoE-layer tokens per second", whole job.  Strong scaling: T is
fixed as N grows.

At N = 1 the line also carries, under "other_workloads", the decode configuration C1 (HBM-bound: achieved GB/s of
algorithmic bytes) and the single-layer prefill configuration C3 (tensor-bound), each with its own roofline entry.

After the timed region rank 0 pushes a few of its token rows through the CPU oracle, layer by layer with the GPU's own
layer inputs and logits, and reports the largest error of the stack under "parity" (every N).

--impl reference times the CPU oracle (the restatement of the reference's arithmetic; the reference ships no CPU or
CUDA implementation of this path) on the host cores, on a bounded sample of the same workload - the same sample, from
the same function, as the "cpu_baseline" leg of the default arm.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=["c0", "c1", "c2", "c3", "c4"])
    ap.add_argument("--layers", type=int, default=0, help="layers resident (default: the configuration's)")
    ap.add_argument("--no-extra", action="store_true", help="skip the C1 / C3 side measurements at N = 1")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-tokens", type=int, default=0, help="tokens of the CPU baseline sample (default by workload)")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiling on a small case)")
    ap.add_argument("--tokens", type=int, default=0, help="override the token count (profiling on a small case)")
    ap.add_argument("--no-graph", action="store_true", help="decode workloads: launch eagerly instead of replaying CUDA graphs")
    ap.add_argument("--micro", type=int, default=0, help="micro-batches per rank in expert-parallel runs (default 1)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--hc-mix", dest="hc_mix", type=int, default=0,
                    help="measure only the hyper-connection mix at this many tokens (tensor-core form from 65 tokens up) and print it")
    ap.add_argument("--parity-rows", type=int, default=32, help="token rows checked against the CPU oracle after the timed region (0 = skip)")
    ap.add_argument("--planes", type=int, default=3, help="BF16 planes of the FP32 router weight on the tensor-core projection (2 or 3)")
    ap.add_argument("--ep", default="native", choices=["native", "torch"],
                    help="expert-parallel driver: the library's C entry point sxb_moe_layer_ep, or torch.distributed (strixite_b200/ep.py)")
    ap.add_argument("--return-path", dest="return_path", type=int, default=None,
                    help="native driver, rows back to their owners: 0 NCCL reduce-scatter, 1 peer stores of FP32 pieces, 2 of F16 pieces "
                         "(default: 1 up to four GPUs, 2 beyond - measured on C4 at eight: F16 pieces 13.0 ms, reduce-scatter 14.3, FP32 pieces 17.5)")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                    help="expert-parallel runs: experts dealt to ranks by calibrated load, or expert e on rank e // (E / N)")
    ap.add_argument("--stage", default="tiles", choices=["tiles", "rows"],
                    help="tcgen05 gate/up activations: gathered once into the tile-blocked form, or converted once and gathered per tile")
    ap.add_argument("--math", default="", help="tcgen05 numerics: wmma_f16 (BF16 per-slot dots, the reference's) or wmma_f16_f32p")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------------------------
# peaks, clocks
# ------------------------------------------------------------------------------------------------------------------

def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.1):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: clocks are reported as unknown, never guessed
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown") else 0x8: "hw_slowdown",
            0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return dict(sm_mhz=(s[len(s) // 2] if s else None), sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                    samples=len(s))


# ------------------------------------------------------------------------------------------------------------------
# the workloads
# ------------------------------------------------------------------------------------------------------------------

class Stack:
    """Resident state of a configuration on this rank: per-layer weights (this rank's experts), router weights, biases,
    the shared workspaces, and the expert-parallel driver."""

    def __init__(self, cfg, layers, seed, dev, rank, world, micro=0, planes=3, ep_impl="native", return_path=1, placement="balanced"):
        import torch
        from strixite_b200 import workloads as W
        from strixite_b200.ep import Compute, ExpertParallelMoe, shard_bounds
        from strixite_b200.layer import MoeBuffers, MoeLayer

        self.cfg, self.n_layers, self.dev, self.rank, self.world = cfg, layers, dev, rank, world
        self.e_lo, self.e_hi = shard_bounds(cfg.E, world, rank)
        self.t_lo, self.t_hi = shard_bounds(cfg.T, world, rank)
        E_local = self.e_hi - self.e_lo
        t = self.t_hi - self.t_lo
        # micro-batches (expert-parallel runs, --micro): chunks of the rank's rows, each with its own work buffers, so that
        # one chunk's all-gather / reduce-scatter runs under the other chunk's GEMMs.  Off by default: measured on C4, the
        # smaller tiles cost the grouped GEMMs more (0.44 -> 0.32 of peak at 8 GPUs) than the overlap returns
        # (19.7 -> 22.9 ms a step at 8 GPUs, 42.2 -> 48.4 ms at 2).
        if micro <= 0 or world == 1 or t % micro != 0:
            micro = 1
        self.micro = micro
        Tc = cfg.T // micro
        self.bufs = [MoeBuffers(Tc, cfg.d, cfg.I, E_local, cfg.k, dev, cfg.shared and world == 1) for _ in range(micro)]
        self.buf = self.bufs[0]
        self.layer_sets = [[] for _ in range(micro)]
        self.wr, self.bias, self.order = [], [], []
        for l in range(layers):
            order = W.expert_placement(cfg, seed, dev, l, world, placement)  # which expert sits where (identity on one GPU)
            w = W.make_layer_weights(cfg, seed, dev, layer=l, e_lo=self.e_lo, e_hi=self.e_hi, order=order)
            for c in range(micro):
                self.layer_sets[c].append(MoeLayer(w, E_local, cfg.k, self.bufs[c], E_total=cfg.E, e_lo=self.e_lo))
            wr, bias = W.placed_router(cfg, seed, dev, l, order)
            self.wr.append(wr)
            self.bias.append(bias)
            self.order.append(order)
        self.layers = self.layer_sets[0]
        # The router-logits projection is the library's: the tensor-core form over the weight split into BF16 planes at
        # load time for prefill-sized batches, the streaming form (the FP32 weight as it is) for decode.
        from strixite_b200 import kernels as K
        self.proj_wmma = t // micro >= 128
        self.planes = [K.router_prepare(w, planes) for w in self.wr] if self.proj_wmma else None
        tc = t // micro
        self.ids_loc = [torch.empty((tc, cfg.k), dtype=torch.int32, device=dev) for _ in range(micro)]
        self.coef_loc = [torch.empty((tc, cfg.k), dtype=torch.float32, device=dev) for _ in range(micro)]
        self.y_part = [torch.empty((Tc, cfg.d), dtype=torch.float32, device=dev) for _ in range(micro)]
        self.logits = [torch.empty((tc, cfg.E + 1), dtype=torch.float32, device=dev) for _ in range(micro)]
        self.router_err = self.buf.router_err
        self.packed = [False] * micro
        self.math = None          # None = by token count (tcgen05 from MoeLayer.tc_min_tokens up)
        self.events = None        # (list, list) of CUDA events around the dominant kernel when roofline timing is on
        self.ep = ExpertParallelMoe(Compute(self._route, self._experts, chunked=True), layers, cfg.T, cfg.d, cfg.k, dev, micro=micro,
                                    exchange="reduce_scatter")
        self.weight_bytes = sum(ly.w.bytes() for ly in self.layers)
        # Expert-parallel runs go through the library's C entry point (sxb_moe_layer_ep: NCCL gathers, this rank's experts,
        # the rows' way back by peer stores or reduce-scatter); --ep torch keeps the torch.distributed driver of ep.py.
        self.native = None
        if world > 1 and ep_impl == "native" and micro == 1:
            import torch.distributed as dist
            box = [K.ep_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            self.native = K.EpContext(box[0], world, rank, cfg.T, cfg.d, cfg.k, return_path)
            self.y_loc = torch.empty((t, cfg.d), dtype=torch.float32, device=dev)

    def layer(self, l, x_loc):
        """One layer on this rank's rows -> y [t, d] FP32."""
        if self.native is None:
            return self.ep.layer(l, x_loc)
        from strixite_b200 import kernels as K
        t = x_loc.shape[0]
        logits = self.logits[0][:t]
        if self.proj_wmma:
            K.router_logits_wmma(x_loc, self.planes[l], self.bias[l], logits)
        else:
            K.router_logits(x_loc, self.wr[l], self.bias[l], logits)
        ly, b = self.layers[l], self.buf
        if b.tiled_x is None:
            b.tiled_x = torch_empty_f16((b.max_tokens * self.cfg.k, self.cfg.d), self.dev)
        self.native.layer(x_loc, logits, self.y_loc, ly.w.gate_up, ly.w.down, ly.E, self.cfg.E, self.e_lo, self.cfg.k, b.ids, b.coef,
                          b.ws, b.ws_bytes, b.h, b.partial, b.router_err, b.expert_err, xs=b.tiled_x,
                          math=ly.math_for(self.cfg.T, self.math))
        return self.y_loc

    def forward(self, x_loc):
        """The stack: x <- bf16(x + moe_l(x)) for every layer."""
        if self.native is None:
            return self.ep.forward(x_loc)
        from strixite_b200.ep import residual
        x = x_loc
        for l in range(self.n_layers):
            x = residual(x, self.layer(l, x))
        return x

    def local_ids(self):
        """The router ids of this rank's own rows after a layer call."""
        if self.world == 1:
            return self.buf.ids
        return self.buf.ids[self.t_lo:self.t_hi] if self.native is not None else self.ids_loc[0]

    def local_slots(self):
        """Slots this rank's experts served in the last layer call (the pack's offsets: the overflow bucket starts there)."""
        from strixite_b200 import kernels as K
        E_local = self.e_hi - self.e_lo
        L = K.route_layout(self.cfg.T, self.cfg.k, E_local)
        return int(self.buf.ws[L["offsets"] + E_local].item())

    def _route(self, l, x_loc, chunk=0):
        from strixite_b200 import kernels as K, workloads as W
        t = x_loc.shape[0]
        logits = self.logits[chunk][:t]
        if self.proj_wmma:
            K.router_logits_wmma(x_loc, self.planes[l], self.bias[l], logits)
        else:
            K.router_logits(x_loc, self.wr[l], self.bias[l], logits)
        buf = self.bufs[chunk]
        if self.world == 1:  # the layer's own routing (router and pack as one launch for a small batch)
            self.packed[chunk] = self.layer_sets[chunk][l].route(logits, t)
            return buf.ids, buf.coef
        ids, coef = self.ids_loc[chunk], self.coef_loc[chunk]
        K.moe_router(logits, logits.stride(0), t, self.cfg.E, self.cfg.k, None, 1, 0, ids, coef, K.Act.F32, buf.router_err)
        return ids, coef

    def _experts(self, l, x_all, ids_all, coef_all, chunk=0):
        layer = self.layer_sets[chunk][l]
        buf = self.bufs[chunk]
        T = x_all.shape[0]
        if self.world > 1:
            buf.ids.copy_(ids_all)
            buf.coef.copy_(coef_all)
        math = layer.math_for(T, self.math)
        y = self.y_part[chunk][:T]
        layer.run_experts(x_all, T, y, math, self.logits[chunk], events=self.events, packed=self.packed[chunk] and self.world == 1)
        return y

    def step(self, x_loc):
        return self.forward(x_loc)

    def one_layer(self, l, x_loc):
        return self.layer(l, x_loc)


def torch_empty_f16(shape, dev):
    import torch
    return torch.empty(shape, dtype=torch.float16, device=dev)


def algorithmic_flops(cfg, layers, shared):
    routed = 2.0 * cfg.T * cfg.k * 3 * cfg.I * cfg.d
    sh = 2.0 * cfg.T * 3 * cfg.I * cfg.d if shared else 0.0
    router = 2.0 * cfg.T * (cfg.E + 1) * cfg.d
    return layers * (routed + sh + router)


def timed(fn, steps, warmup, dist_on, dev):
    """W untimed steps, then exactly K steps between a barrier + synchronize on both sides; CUDA events on the current
    stream; the maximum over ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def kernel_ms(events):
    """Average duration (ms) of the dominant kernel from the CUDA events recorded around each of its launches."""
    starts, ends = events
    if not starts:
        return None
    return sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / len(starts)


def run_stack(cfg, args, dev, rank, world, peaks, layers=None, rotate=False):
    """Times a configuration.  rotate: a step runs ONE layer, cycling through the resident layers so consecutive steps
    never find their weights in L2 (decode); otherwise a step runs the whole stack."""
    import torch
    import torch.distributed as dist
    from strixite_b200 import kernels as K, workloads as W

    layers = layers or args.layers or cfg.layers
    st = Stack(cfg, layers, args.seed, dev, rank, world, micro=getattr(args, "micro", 0), planes=getattr(args, "planes", 3),
               ep_impl=getattr(args, "ep", "native"), return_path=getattr(args, "return_path", 1),
               placement=getattr(args, "placement", "balanced"))
    if getattr(args, "stage", "tiles") == "rows":
        for ls in st.layer_sets:
            for ly in ls:
                ly.stage_rows = True
    if getattr(args, "math", ""):
        from strixite_b200.kernels import MoeMath
        st.math_tc = {"wmma_f16": MoeMath.WmmaF16, "wmma_f16_f32p": MoeMath.WmmaF16F32Partials}[args.math]
        for ls in st.layer_sets:
            for ly in ls:
                ly.tc_math = st.math_tc
    t_loc = st.t_hi - st.t_lo
    x_full = W.activations(cfg, args.seed, dev)
    x_loc = x_full[st.t_lo:st.t_hi].contiguous()
    x_host = x_loc.cpu().pin_memory()
    x_dev = torch.empty_like(x_loc)
    y_host = torch.empty((t_loc, cfg.d), dtype=torch.bfloat16).pin_memory()
    counter = {"i": 0}

    def device_step():
        if rotate:
            st.one_layer(counter["i"] % layers, x_loc)
            counter["i"] += 1
        else:
            st.step(x_loc)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        if rotate:
            y = st.one_layer(counter["i"] % layers, x_dev)
            counter["i"] += 1
            y_host.copy_(y.to(torch.bfloat16), non_blocking=True)
        else:
            y_host.copy_(st.step(x_dev), non_blocking=True)

    dist_on = world > 1
    K.LAUNCHES = 0
    device_step()
    torch.cuda.synchronize()
    launches_per_step = K.LAUNCHES
    K.check_router_error(st.router_err, cfg.name)
    for ly in st.layers[:1]:
        ly.check_errors(cfg.name)

    graphs = None
    if rotate and world == 1 and not args.no_graph:
        # Decode: a layer is eight short launches, and the gaps between them are a tenth of the step.  Every layer's launch
        # sequence (all of it goes to the caller's stream through the C ABI) is captured once into a CUDA graph over static
        # buffers and replayed; the kernels and their arguments are those of the eager path.
        for l in range(layers):  # every layer eagerly once more: lazy initialisation must not fall inside a capture
            st.one_layer(l, x_dev)
        torch.cuda.synchronize()
        x_dev.copy_(x_loc)
        graphs = []
        for l in range(layers):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                y_l = st.one_layer(l, x_dev)
            graphs.append((g, y_l))

        def device_step():  # noqa: F811  (replaces the eager step above)
            graphs[counter["i"] % layers][0].replay()
            counter["i"] += 1

        def e2e_step():  # noqa: F811
            x_dev.copy_(x_host, non_blocking=True)
            g, y_l = graphs[counter["i"] % layers]
            g.replay()
            counter["i"] += 1
            y_host.copy_(y_l.to(torch.bfloat16), non_blocking=True)

    with ClockSampler(dev.index or 0) as clocks:
        st.events = ([], [])
        ms = timed(device_step, args.steps, args.warmup, dist_on, dev)
        ev = st.events
        st.events = None
        # the events recorded during warm-up are dropped: keep those of the timed steps only
        per_step = len(ev[0]) // (args.steps + args.warmup) if ev[0] else 0
        ev = (ev[0][per_step * args.warmup:], ev[1][per_step * args.warmup:])
        k_ms = kernel_ms(ev)
        e2e_ms = timed(e2e_step, args.steps, 1, dist_on, dev)
        if graphs is not None:  # the dominant kernel's own time: a few eager layers with events around it
            st.events = ([], [])
            for i in range(2 * layers):
                st.one_layer(i % layers, x_loc)
            torch.cuda.synchronize()
            k_ms = kernel_ms((st.events[0][layers:], st.events[1][layers:]))
            st.events = None
    ep_info = None
    if world > 1:
        # per rank: the phases of a layer (ms, mean over one more pass of the stack) and the slots its experts served
        if st.native is not None:
            st.native.set_timing(True)
            st.step(x_loc)
            phases = st.native.timing()
            st.native.set_timing(False)
        else:
            st.ep.timing = []
            st.step(x_loc)
            phases = st.ep.timing_summary() or {}
            st.ep.timing = None
        slots, x_l = [], x_loc
        from strixite_b200.ep import residual
        for l in range(layers):
            y_l = st.layer(l, x_l)
            slots.append(st.local_slots())
            x_l = residual(x_l, y_l)
        mine = {"rank": rank, "phases_ms": phases, "slots_per_layer": slots}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        ep_info = gathered
    layer_tokens = cfg.T * (1 if rotate else layers)
    out = dict(
        ms_per_step=ms, value=layer_tokens / (ms * 1e-3), e2e_value=layer_tokens / (e2e_ms * 1e-3), e2e_ms=e2e_ms,
        h2d=x_host.numel() * 2 * world, d2h=y_host.numel() * 2 * world, launches=launches_per_step, clocks=clocks.summary(),
        kernel_ms=k_ms, layers=layers, stack=st, x_full=x_full, ep_info=ep_info,
    )
    return out


def roofline_ep(cfg, res, peaks, world):
    """Expert-parallel runs: every rank's own expert phase (pack, activation staging, gate/up + SwiGLU, down, combine - the
    CUDA events of sxb_moe_layer_ep around it) against the flops of the slots that rank's experts served."""
    per_rank = []
    for info in res["ep_info"]:
        ms = info["phases_ms"].get("experts")
        slots = sum(info["slots_per_layer"]) / max(1, len(info["slots_per_layer"]))
        flops = 2.0 * slots * 3 * cfg.I * cfg.d
        per_rank.append({"rank": info["rank"], "slots_per_layer": slots, "experts_ms": ms,
                         "tflops": (flops / (ms * 1e-3) / 1e12) if ms else None})
    mine = per_rank[0]
    peak = peaks["tflops_sustained"]
    return dict(bound="tensor", kernel="experts phase of sxb_moe_layer_ep (pack, staging, gate/up + SwiGLU, down, combine), rank 0",
                achieved=mine["tflops"], peak=peak, unit="TFLOP/s", frac=(mine["tflops"] / peak) if mine["tflops"] else None,
                peak_source=peaks["source"] + " (sustained bf16)", traffic=None, per_rank=per_rank,
                flops_per_launch=2.0 * mine["slots_per_layer"] * 3 * cfg.I * cfg.d, kernel_ms=mine["experts_ms"])


def roofline_tensor(cfg, res, peaks, world):
    """Dominant kernel of the prefill regime: the grouped gate/up + SwiGLU GEMM, 2 * S * 2I * d flops per launch (this
    rank's share of the slots: S / N on average)."""
    if world > 1 and res.get("ep_info") and res["ep_info"][0]["phases_ms"].get("experts"):
        return roofline_ep(cfg, res, peaks, world)
    micro = res["stack"].micro  # a launch serves one micro-batch of this rank's slots
    flops = 2.0 * cfg.T * cfg.k * 2 * cfg.I * cfg.d / world / micro
    if not res["kernel_ms"]:
        return None
    achieved = flops / (res["kernel_ms"] * 1e-3) / 1e12
    peak = peaks["tflops_sustained"]
    # DRAM bytes of one launch: an ncu capture of a reduced case (64 experts, 512 tokens) read 328.0 MB against 327.1 MB of
    # codes + scales / mins + tile-blocked activations, a ratio of 1.00; the same sum for this launch, times that ratio.
    ly = res["stack"].layers[0]
    traffic = 1.003 * (ly.w.gate_up.bytes() + cfg.T * cfg.k / world / micro * cfg.d * 2)
    # which tcgen05 kernel serves gate/up (launch_tc in csrc/grouped_tc.cu): tile-blocked activations and >= 160 slots an expert
    # on average go to the 128-row x 256-token kernel, fewer stay on the 256-row x 128-token one
    name = "tiled_tc_kernel" if cfg.T * cfg.k / world / micro / (cfg.E / world) >= 160 else "grouped_tc_kernel"
    return dict(bound="tensor", kernel=name + "<gate_up+swiglu>", achieved=achieved, peak=peak, unit="TFLOP/s",
                frac=achieved / peak, peak_source=peaks["source"] + " (sustained bf16)",
                frac_of_burst=achieved / peaks["tflops_burst"], peak_burst=peaks["tflops_burst"], traffic=traffic,
                traffic_source="dram bytes of an ncu capture of a reduced case, scaled by algorithmic bytes",
                flops_per_launch=flops, kernel_ms=res["kernel_ms"])


def decode_bytes(cfg, stack, layer_idx):
    """Algorithmic bytes of one decode layer: every DISTINCT routed expert's gate/up and down once, the shared expert,
    the router weight, x in and y out."""
    import torch
    ly = stack.layers[layer_idx]
    ids = stack.buf.ids[: cfg.T]
    U = int(torch.unique(ids).numel())
    per_expert = ly.w.gate_up.bytes() // ly.E + ly.w.down.bytes() // ly.E
    b = U * per_expert
    gu_b = U * (ly.w.gate_up.bytes() // ly.E)
    if ly.w.shared_gate_up is not None:
        b += ly.w.shared_gate_up.bytes() + ly.w.shared_down.bytes()
    b += (cfg.E + 1) * cfg.d * 4 + 2 * cfg.T * cfg.d * 2
    return b, U, gu_b


def decode_bytes_mean(cfg, res):
    """decode_bytes averaged over the resident layers (they differ in which experts their tokens pick)."""
    import torch
    st = res["stack"]
    x = res["x_full"][st.t_lo:st.t_hi].contiguous()
    per_layer = []
    for l in range(res["layers"]):
        st.one_layer(l, x)
        torch.cuda.synchronize()
        per_layer.append(decode_bytes(cfg, st, l))
    n = len(per_layer)
    return sum(p[0] for p in per_layer) / n, sum(p[1] for p in per_layer) / n, sum(p[2] for p in per_layer) / n


def config_dict(cfg, layers, world, micro=1, extra=None):
    """The workload's description, the same keys on every arm."""
    d = {"workload": cfg.name, "T": cfg.T, "layers": layers, "hidden": cfg.d, "experts": cfg.E, "experts_per_gpu": cfg.E // world,
         "top_k": cfg.k, "intermediate": cfg.I, "gate_up": f"q{cfg.gu_bits}g{cfg.group(cfg.gu_bits)}",
         "down": f"q{cfg.dn_bits}g{cfg.group(cfg.dn_bits)}", "shared_expert": cfg.shared, "expert_bias": cfg.bias,
         "parallelism": f"ep{world}" + (f", {micro} micro-batches a rank" if micro > 1 else ""), "value_is": "T * layers / step time"}
    d.update(extra or {})
    return d


def semantics_of(cfg, math=None):
    if cfg.T < 256:
        return "decode"
    return "grouped_f32_partials" if (math is not None and int(math) == 6) else "grouped"


def cpu_sample(cfg, seed, n_tokens, semantics, dev, repeats=1, warmup=0):
    """The CPU oracle on the first n_tokens rows of layer 0 of the workload, on all host cores: inputs drawn as the GPU arm
    draws them (same generators, same seed), router logits formed on the host in float64, the experts those rows pick
    regenerated and quantized expert by expert.  Returns (seconds per pass, oracle output, cores).  Only the oracle's
    moe_layer is timed."""
    import numpy as np
    from oracle import check, cpu
    from strixite_b200 import workloads as W
    cpu.build(None)
    x = W.activations(cfg, seed, dev)[:n_tokens]
    xb = check.bits_of(x)
    wr = W.router_weight(cfg, seed, dev).cpu().numpy().astype(np.float64)
    bias = W.expert_bias(cfg, seed, dev).cpu().numpy().astype(np.float64)
    logits = (cpu.bf16_to_f32(xb).astype(np.float64) @ wr.T + bias).astype(np.float32)
    shared = None
    if cfg.shared:
        import torch
        def one(which):
            w32 = W.expert_weight_f32(cfg, seed, dev, which, 0, 0)
            if torch.device(dev).type == "cuda":
                from strixite_b200 import kernels as K
                return check.download(K.quantize(w32, 64, 8), cpu)
            return cpu.quantize(w32.numpy(), 64, 8)
        shared = (one("shared_gate_up"), one("shared_down"))
    times, out = [], None
    real = cpu.moe_layer

    def stamped(*a, **k):
        t0 = time.perf_counter()
        r = real(*a, **k)
        times.append(time.perf_counter() - t0)
        return r

    fetched = {}
    gen = check.generated_experts(cfg, seed, 0, dev)

    def fetch(which, experts):  # the weights are generated once, outside the timed call, and reused by every pass
        key = (which, tuple(int(e) for e in experts))
        if key not in fetched:
            fetched[key] = gen(which, experts)
        return fetched[key]

    cpu.moe_layer = stamped
    try:
        for _ in range(warmup + repeats):
            out = check.oracle_layer_with(cpu, cfg, fetch, shared, xb, logits, semantics)
    finally:
        cpu.moe_layer = real
    kept = times[warmup:]
    return sum(kept) / len(kept), out, cpu.hardware_threads()


def cpu_tokens(cfg, args):
    """Size of the CPU sample: every token of a decode workload, 768 rows of a prefill one (seconds of host work)."""
    return args.cpu_tokens or (cfg.T if cfg.T <= 64 else 768)


def cpu_baseline(cfg, args, dev):
    n = cpu_tokens(cfg, args)
    sem = semantics_of(cfg)
    sec, _, cores = cpu_sample(cfg, args.seed, n, sem, dev)
    return dict(value=n / sec, unit="MoE-layer tokens/s", cores=cores, kind="port",
                sample=f"{n} tokens of layer 0 of {cfg.name} through the CPU oracle ({sem} semantics), {sec:.2f} s a pass")


def parity_check(cfg, st, x_loc, args, dev, rank):
    """Rank 0, after the timed region: `rows` of this rank's token rows through the CPU oracle for EVERY layer of the stack,
    each layer fed the GPU's own input rows and router logits of that layer (so that a rounding difference in one layer
    does not turn into different routing in the next: the layers are checked one by one, all of them).  Returns the
    largest max|y - y_ref| / rms(y_ref) over the layers, layer 0's, and whether every layer's router ids are the
    oracle's for those logits."""
    import numpy as np
    import torch
    from oracle import check, cpu
    from strixite_b200.ep import residual
    cpu.build(None)
    n = min(args.parity_rows, x_loc.shape[0])
    g = torch.Generator(device="cpu").manual_seed(args.seed + 17)
    rows = torch.sort(torch.randperm(x_loc.shape[0], generator=g)[:n]).values.to(dev)
    sem = semantics_of(cfg, st.layers[0].math_for(cfg.T, st.math))
    rec = []
    x = x_loc
    for l in range(st.n_layers):
        y = st.layer(l, x)
        ids = st.local_ids()
        rec.append((check.bits_of(x[rows]), st.logits[0][rows].cpu().numpy(), ids[rows].cpu().numpy(), y[rows].float().cpu().numpy()))
        x = residual(x, y)
    torch.cuda.synchronize()
    if rank != 0:  # every rank runs the forward (its collectives); rank 0 alone consults the oracle
        return None
    worst, first, ids_ok = 0.0, None, True
    for l, (xb, lg, ids, y) in enumerate(rec):
        shared = None
        if cfg.shared:
            w = st.layers[l].w
            shared = (check.download(w.shared_gate_up, cpu), check.download(w.shared_down, cpu))
        ref = check.oracle_layer_with(cpu, cfg, check.generated_experts(cfg, args.seed, l, dev, st.order[l]), shared, xb, lg, sem)
        ids_ok = ids_ok and bool(np.array_equal(ref["ids"], ids))
        err = check.max_abs_over_rms(y, ref["y_f32"])
        worst = max(worst, err)
        if l == 0:
            first = err
    return {"rows": int(n), "layers": st.n_layers, "max_abs_over_rms": worst, "layer0": first, "ids_exact": ids_ok,
            "tolerance": 1e-2, "semantics": sem,
            "how": "every layer of the stack against the CPU oracle on the GPU's own layer inputs and logits; rank 0's rows"}


def run_reference(args):
    """--impl reference: the CPU oracle on the host cores, the same bounded sample of the same seeded layer as the default
    arm's cpu_baseline leg, once per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from strixite_b200 import workloads as W
    cfg = W.c2_config(args.seed) if args.workload == "c2" else W.CONFIGS[args.workload]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    n_tok = cpu_tokens(cfg, args)
    if dev.type == "cpu" and not args.cpu_tokens:
        n_tok = min(n_tok, 16)  # no GPU to draw and quantize the experts on: keep the host-side generation short
    sem = semantics_of(cfg)
    sec, _, cores = cpu_sample(cfg, args.seed, n_tok, sem, dev, repeats=args.steps, warmup=min(args.warmup, 1))
    value = n_tok / sec
    unit = "MoE-layer tokens/s"
    layers = args.layers or (8 if cfg.T <= 64 else cfg.layers)
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 accumulate, bf16 activations", "data": "synthetic",
        "config": config_dict(cfg, layers, max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port",
                         "sample": f"{n_tok} tokens of layer 0 of {cfg.name} through the CPU oracle ({sem} semantics) per step, "
                                   f"{sec:.2f} s a pass (the reference has no CPU or CUDA implementation of this path; this is "
                                   f"the CPU oracle restating its arithmetic)"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def hc_mix_measure(dev, peaks, seed, T=16, d=4096, r=320, H=4, iters=50):
    """The hyper-connection mix that produces the block's input (hc_mix_down + hc_mix_up, Q8 g64 weights) at the decode
    configuration's T and d: microseconds a mix (CUDA events, the 10.6 MB of weights rotated through eight copies so that
    every mix reads them from HBM) and the bandwidth that is of the measured peak."""
    import torch
    from strixite_b200 import kernels as K
    g = torch.Generator(device=dev).manual_seed(seed + 77)
    copies = []
    for _ in range(8):
        wd_f = torch.randn((r + H, H * d), device=dev, generator=g) * 0.05
        wu_f = torch.randn((H * d, r), device=dev, generator=g) * 0.2
        copies.append((K.quantize(wd_f, 64, 8), K.to_chunk_major(K.quantize(wu_f, 64, 8))))
    x = torch.randn((T, H * d), device=dev, generator=g).to(torch.bfloat16)
    norm_w = torch.randn(H * d, device=dev, generator=g) * 0.1
    h = torch.empty((T, r), dtype=torch.float32, device=dev)
    w_in, inv = torch.empty((T, H), dtype=torch.float32, device=dev), torch.empty((T, H), dtype=torch.float32, device=dev)
    u = torch.empty((T, d), dtype=torch.bfloat16, device=dev)

    def mix(i):
        wd, wu = copies[i % len(copies)]
        K.hc_mix_down(x, wd, T, H, d, r, True, 1e-6, h, w_in, inv, K.Act.BF16)
        K.hc_mix_up(h, wu, x, norm_w, inv, T, H, d, u, K.Act.BF16)

    for i in range(8):
        mix(i)
    torch.cuda.synchronize()
    # eight mixes (one per weight copy) as one CUDA graph, as the decode layers are timed: two launches of tens of
    # microseconds each are otherwise timed by the host's launch rate, not by the GPU
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(len(copies)):
            mix(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, iters // len(copies))
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * len(copies))
    nbytes = copies[0][0].bytes() + copies[0][1].bytes() + 2 * x.numel() * 2 + u.numel() * 2
    gbs = nbytes / (us * 1e-6) / 1e9
    return {"T": T, "d": d, "r": r, "weights": "q8g64", "us_per_mix": us, "bytes_per_mix": nbytes, "launches_per_mix": 2,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]}}


def hc_mix_prefill_measure(dev, peaks, seed, T=4096, d=4096, r=320, H=4, iters=10):
    """The same mix for a multi-token forward on the tensor cores (hc_mix_down_wmma + hc_mix_up_wmma, Q8 g64 weights):
    milliseconds a mix by CUDA events, each half on its own as well, and the products' 2 T H d (R + r) flops against the
    measured bf16 peak.  The streams X (T H d BF16, 134 MB at the default) are larger than L2."""
    import torch
    from strixite_b200 import kernels as K
    g = torch.Generator(device=dev).manual_seed(seed + 78)
    R = r + H
    wd = K.quantize(torch.randn((R, H * d), device=dev, generator=g) * 0.05, 64, 8)
    wu = K.to_chunk_major(K.quantize(torch.randn((H * d, r), device=dev, generator=g) * 0.2, 64, 8))
    x = torch.randn((T, H * d), device=dev, generator=g).to(torch.bfloat16)
    norm_w = torch.randn(H * d, device=dev, generator=g) * 0.1
    h = torch.empty((T, r), dtype=torch.float32, device=dev)
    w_in, inv = torch.empty((T, H), dtype=torch.float32, device=dev), torch.empty((T, H), dtype=torch.float32, device=dev)
    u = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
    ws_d = torch.empty(K.hc_wmma_workspace_bytes(T, H, d, R, 8, 64), dtype=torch.uint8, device=dev)
    ws_u = torch.empty(K.hc_mix_up_wmma_workspace_bytes(T, H, d, r, 8, 64), dtype=torch.uint8, device=dev)

    def down():
        K.hc_mix_down_wmma(x, wd, T, H, d, r, True, 1e-6, h, w_in, inv, ws_d, K.Act.BF16)

    def up():
        K.hc_mix_up_wmma(h, wu, x, norm_w, inv, T, H, d, u, ws_u, K.Act.BF16)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ms_down, ms_up = timed(down), timed(up)
    ms = timed(lambda: (down(), up()))
    K.check_grouped_status(ws_d, "hc_mix_down_wmma")
    K.check_dense_status("hc_mix_up_wmma")
    flops = 2.0 * T * H * d * (R + r)
    tf = flops / (ms * 1e-3) / 1e12
    return {"T": T, "d": d, "r": r, "weights": "q8g64", "ms_per_mix": ms, "ms_down": ms_down, "ms_up": ms_up,
            "launches_per_mix": 8,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops_burst"], "unit": "TFLOP/s", "frac": tf / peaks["tflops_burst"]},
            "hbm_bytes_floor": 2 * x.numel() * 2 + u.numel() * 2}


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    from strixite_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU implementation (see --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    peaks = measured_peaks()
    if args.hc_mix:
        m = hc_mix_prefill_measure(dev, peaks, args.seed, T=args.hc_mix) if args.hc_mix > 64 else hc_mix_measure(dev, peaks, args.seed, T=args.hc_mix)
        print(json.dumps({"metric": "hyper-connection mix", "n_gpus": 1, **m}))
        return
    cfg = W.c2_config(args.seed) if args.workload == "c2" else W.CONFIGS[args.workload]
    if args.experts or args.tokens:
        from dataclasses import replace
        cfg = replace(cfg, E=args.experts or cfg.E, T=args.tokens or cfg.T, name=cfg.name + "_reduced")
    decode = cfg.T <= 64

    if args.return_path is None:
        args.return_path = 1 if world <= 4 else 2
    if cfg.shared and world > 1:
        raise SystemExit(f"{cfg.name} has a shared expert, which is not sharded: run it on one GPU (the expert-parallel workload is c4)")
    res = run_stack(cfg, args, dev, rank, world, peaks, layers=(8 if decode else None), rotate=decode)
    st = res["stack"]
    line = {
        "metric": "moe_layer_tokens_per_s", "value": res["value"], "unit": "MoE-layer tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 x f16 -> f32 (tcgen05), bf16 activations" if not decode
        else "bf16 x int4/int8 codes -> f32 (mma.sync), bf16 activations",
        "data": "synthetic",
        "config": config_dict(cfg, res["layers"], world, st.micro),
        "details": {
            "router_projection": ("sxb_router_logits_wmma (tcgen05, FP32 weight as %d BF16 planes)" % args.planes) if st.proj_wmma
            else "sxb_router_logits (streaming, FP32 weight)",
            "residual": "sxb_residual_add",
            "l2": "weights resident per step exceed L2 (126 MB): %.1f GB on this rank" % (st.weight_bytes / 1e9)},
        "clocks": res["clocks"], "gpu_launches": res["launches"],
        "e2e": {"value": res["e2e_value"], "unit": "MoE-layer tokens/s", "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"], "ms_per_step": res["e2e_ms"]},
    }
    if res.get("ep_info"):
        line["expert_parallel"] = {"driver": "sxb_moe_layer_ep" if st.native is not None else "torch.distributed (ep.py)",
                                   "return_path": {0: "nccl reduce-scatter (fp32)", 1: "peer stores, fp32 pieces", 2: "peer stores, f16 pieces"}[args.return_path]
                                   if st.native is not None else st.ep.exchange, "placement": args.placement, "per_rank": res["ep_info"]}
    if args.parity_rows > 0:
        try:
            par = parity_check(cfg, st, res["x_full"][st.t_lo:st.t_hi].contiguous(), args, dev, rank)
        except Exception as e:  # a checker failure must not lose the measured line; it is reported as such
            par = {"rows": 0, "error": f"{type(e).__name__}: {e}"}
            if world > 1:
                raise
        if par is not None:
            line["parity"] = par
    if decode:
        b, U, gu_b = decode_bytes_mean(cfg, res)
        line["roofline"] = dict(bound="hbm", kernel="whole layer", achieved=b / (res["ms_per_step"] * 1e-3) / 1e9,
                                peak=peaks["hbm_gbs"], unit="GB/s", frac=b / (res["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                peak_source=peaks["source"], traffic=b,
                                traffic_source="ncu: the stream kernels' dram bytes equal their algorithmic bytes (610.7 of 610 MB)",
                                bytes_per_launch=b, distinct_experts=U)
    else:
        line["roofline"] = roofline_tensor(cfg, res, peaks, world)
        line["achieved_tflops_whole_step"] = algorithmic_flops(cfg, res["layers"], cfg.shared and world == 1) / (res["ms_per_step"] * 1e-3) / 1e12

    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            line["cpu_baseline"] = cpu_baseline(cfg, args, dev)
        except Exception as e:  # the baseline is a reported extra: never lose the GPU line to it
            line["cpu_baseline"] = {"value": None, "unit": "MoE-layer tokens/s", "cores": None, "kind": "port",
                                    "sample": f"failed: {type(e).__name__}: {e}"}
    del res, st

    if rank == 0 and world == 1 and not args.no_extra and args.workload == "c4":
        extra = {}
        torch.cuda.empty_cache()
        for name in ("c1", "c3"):
            c = W.CONFIGS[name]
            dec = c.T <= 64
            r = run_stack(c, args, dev, 0, 1, peaks, layers=(8 if dec else 1), rotate=dec)
            e = {"tokens_per_s": r["value"], "ms_per_step": r["ms_per_step"], "e2e_tokens_per_s": r["e2e_value"],
                 "gpu_launches": r["launches"], "clocks": r["clocks"]}
            if args.parity_rows > 0:
                try:
                    e["parity"] = parity_check(c, r["stack"], r["x_full"], args, dev, 0)
                except Exception as ex:
                    e["parity"] = {"rows": 0, "error": f"{type(ex).__name__}: {ex}"}
            if dec:
                b, U, gu_b = decode_bytes_mean(c, r)
                gbs = b / (r["ms_per_step"] * 1e-3) / 1e9
                e["roofline"] = dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"],
                                     bytes_per_step=b, distinct_experts=U, peak_source=peaks["source"])
                if r["kernel_ms"]:
                    e["roofline"]["gate_up_kernel"] = dict(ms=r["kernel_ms"], gbs=gu_b / (r["kernel_ms"] * 1e-3) / 1e9,
                                                           frac=gu_b / (r["kernel_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"])
            else:
                e["roofline"] = roofline_tensor(c, r, peaks, 1)
                e["achieved_tflops_whole_step"] = algorithmic_flops(c, 1, c.shared) / (r["ms_per_step"] * 1e-3) / 1e12
            extra[c.name] = e
            del r
            torch.cuda.empty_cache()
        try:
            extra["hc_mix_decode"] = hc_mix_measure(dev, peaks, args.seed)
        except Exception as ex:
            extra["hc_mix_decode"] = {"error": f"{type(ex).__name__}: {ex}"}
        try:
            extra["hc_mix_prefill"] = hc_mix_prefill_measure(dev, peaks, args.seed)
        except Exception as ex:
            extra["hc_mix_prefill"] = {"error": f"{type(ex).__name__}: {ex}"}
        line["other_workloads"] = extra

    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
