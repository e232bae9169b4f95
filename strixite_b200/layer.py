"""The MoE sublayer as the reference's forward composes it (runtime/qwen4exp.cpp:3143-3217), over the C ABI.

    router top-k  ->  shared expert (dense Q8 gate_up, SwiGLU, down)  ->  pack slots by expert
                  ->  grouped gate/up + SwiGLU  ->  grouped down, combine, + sigmoid(gate) * shared

`MoeLayer` owns what the reference's session owns for this block (runtime/qwen4exp.cpp:1018-1027,1092-1101): ids,
coef, the grouping workspace, h, the combine's partial, the shared expert's buffers and the two error buffers.
Everything is enqueued on the current CUDA stream; nothing synchronizes except `check_errors`.

Path choice by token count (the reference's kGroupedMinTokens / kWideMin*, runtime/qwen4exp.hpp:724):
    T <  tc_min_tokens : exact-product streaming kernels (HBM-bound regime; MoeMath.F32)
    T >= tc_min_tokens : tcgen05 grouped GEMMs (MoeMath.WmmaF16)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import kernels as K
from .kernels import Act, MoeMath, QDeviceView


@dataclass
class MoeWeights:
    """runtime/qwen4exp.hpp:129-132 Layer{gate_up, down, shared_gate_up, shared_down}; experts stacked along N."""

    gate_up: QDeviceView                       # [E * 2I, d]
    down: QDeviceView                          # [E * d, I]
    shared_gate_up: Optional[QDeviceView] = None  # [2I, d]
    shared_down: Optional[QDeviceView] = None     # [d, I]

    def bytes(self) -> int:
        n = self.gate_up.bytes() + self.down.bytes()
        if self.shared_gate_up is not None:
            n += self.shared_gate_up.bytes() + self.shared_down.bytes()
        return n


class MoeBuffers:
    """Workspaces for up to max_tokens tokens; shared by every layer of a stack (the reference's session buffers)."""

    def __init__(self, max_tokens: int, d: int, I: int, E_buckets: int, A: int, device, shared: bool):
        T, S = max_tokens, max_tokens * A
        dev = device
        self.max_tokens, self.A = T, A
        self.ids = torch.empty((T, A), dtype=torch.int32, device=dev)
        self.coef = torch.empty((T, A), dtype=torch.float32, device=dev)
        self.ws_bytes = K.moe_route_workspace_bytes(T, A, E_buckets)
        self.ws = torch.empty(self.ws_bytes // 4, dtype=torch.int32, device=dev)
        self.h = torch.empty((S, I), dtype=torch.bfloat16, device=dev)
        self.partial = torch.empty((S, d), dtype=torch.float32, device=dev)
        self.side_stream = None  # second stream for the shared expert in the decode regime (made on first use)
        self.tiled_x = None     # x in tile-blocked F16 form for the routed experts (tcgen05 path), made on first use
        self.tiled_x_sh = None  # the same for the shared expert's single bucket
        self.router_err = torch.zeros(4, dtype=torch.int32, device=dev)
        self.expert_err = torch.zeros(4, dtype=torch.int32, device=dev)
        if shared:
            self.sh_gu = torch.empty((T, 2 * I), dtype=torch.bfloat16, device=dev)
            self.sh_h = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
            self.sh_y = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
            self.sh_y32 = torch.empty((T, d), dtype=torch.float32, device=dev)


class MoeLayer:
    """One MoE sublayer.  E_total / e_lo: expert-parallel ranks hold experts [e_lo, e_lo + E_local) of E_total in their
    weight views and return their partial sum of y (see `ep.ExpertParallelMoe`)."""

    tc_min_tokens = 256
    # The tcgen05 path's numerics.  WmmaF16F32Partials keeps the combine's per-slot dots in FP32; WmmaF16 rounds them to
    # BF16 as the reference's served path does, which by itself moves an output by up to ~2e-2 of the output RMS
    # (measured on the Zipf-routed stack) - beyond the 1e-2 this path is held to - and measured no faster here.
    tc_math = MoeMath.WmmaF16F32Partials
    stage_rows = False          # tcgen05 path: True = x converted once to F16 rows (sxb_stage_f16) and gathered per tile by the
                                # kernel's copy warps; False = x gathered once into the tile-blocked form (sxb_stage_f16_tiles)
    small_slots = 2048          # up to this many slots the router and the pack are one launch (sxb_moe_route_small)

    def __init__(self, weights: MoeWeights, n_experts: int, top_k: int, buffers: MoeBuffers, E_total: Optional[int] = None,
                 e_lo: int = 0):
        self.w = weights
        self.E = n_experts                      # experts in the weight views
        self.E_total = n_experts if E_total is None else E_total
        self.e_lo = e_lo
        self.k = top_k
        self.buf = buffers
        self.d = weights.gate_up.K
        self.I = weights.gate_up.N // n_experts // 2
        assert weights.down.N == n_experts * self.d and weights.down.K == self.I
        self.ep = self.E_total != self.E

    def math_for(self, T: int, math: Optional[MoeMath]) -> MoeMath:
        if math is not None:
            return math
        return self.tc_math if T >= self.tc_min_tokens else MoeMath.F32

    def route(self, logits: torch.Tensor, T: int) -> bool:
        """moe_router on logits [T, ld] FP32 (column E_total = the shared gate when ld > E_total).  For a small batch the
        pack rides in the same launch; returns whether it did."""
        b = self.buf
        if T * self.k <= self.small_slots and not self.ep:
            K.moe_route_small(logits, logits.stride(0), T, self.E_total, self.k, 0, self.E, b.ids, b.coef, b.ws, b.ws_bytes,
                              b.router_err, b.expert_err)
            return True
        K.moe_router(logits, logits.stride(0), T, self.E_total, self.k, None, 1, 0, b.ids, b.coef, Act.F32, b.router_err)
        return False

    def shared_expert(self, x: torch.Tensor, T: int, math: MoeMath, out: torch.Tensor):
        """The always-on shared expert as dense projections -> out [T, d] (runtime/qwen4exp.cpp:3163-3168): BF16 as the
        reference stores it, or FP32 (the unrounded sums) when the layer's output is asked for in FP32."""
        b, w = self.buf, self.w
        out_act = Act.F32 if out.dtype == torch.float32 else Act.BF16
        if not K_is_f16(math):
            K.linear_qw(x, w.shared_gate_up, b.sh_gu, T, Act.BF16)
            K.swiglu(b.sh_gu, b.sh_h, T, self.I, Act.BF16)
            K.linear_qw(b.sh_h, w.shared_down, out, T, Act.BF16, out_act)
            return
        # Prefill: dense projections on the tcgen05 kernel (kernels/linear_wmma.hip:69-113), SwiGLU fused into the first
        if b.tiled_x_sh is None:
            b.tiled_x_sh = torch.empty((b.max_tokens, self.d), dtype=torch.float16, device=x.device)
        K.stage_f16_tiles(x, None, 0, T, 1, 1, self.d, w.shared_gate_up.bits, b.tiled_x_sh)
        hf = 3 if w.shared_down.bits == 4 else 4
        K.linear_qw_wmma_swiglu(b.tiled_x_sh, w.shared_gate_up, b.sh_h, T, Act.F16_TILED, h_f16=hf)
        K.linear_qw_wmma(b.sh_h, w.shared_down, out, T, Act.F16_TILED, out_act)

    def experts(self, x: torch.Tensor, T: int, y: torch.Tensor, math: MoeMath, gate_logit=None, gate_ld: int = 0,
                shared_out: Optional[torch.Tensor] = None, events=None, before_combine=None, packed: bool = False):
        """pack -> gate/up + SwiGLU -> down + combine into y [T, d] (BF16 or FP32), ids / coef already in the buffers
        (packed: the workspace too)."""
        b, w, A = self.buf, self.w, self.k
        out_act = Act.F32 if y.dtype == torch.float32 else Act.BF16
        if packed:
            pass
        elif self.ep:
            K.moe_group_routes_ep(b.ids, T, A, self.E_total, self.e_lo, self.E, b.ws, b.ws_bytes, b.expert_err)
        else:
            K.moe_group_routes(b.ids, T, A, self.E, b.ws, b.ws_bytes, b.expert_err)
        if events is not None:  # CUDA events around the dominant kernel (the benchmark's roofline timing)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        tc = K_is_f16(math)
        hf = (3 if w.down.bits == 4 else 4) if tc else 0
        if tc:
            # x gathered into the tile-blocked F16 form once; every row block of every tile then bulk-copies its operand
            if b.tiled_x is None:
                b.tiled_x = torch.empty((b.max_tokens * A, self.d), dtype=torch.float16, device=x.device)
            if self.stage_rows:
                K.stage_f16(x, T, self.d, w.gate_up.bits, b.tiled_x)
                K.linear_qw_experts_gather_grouped_swiglu(b.tiled_x, w.gate_up, self.E, b.ws, b.ws_bytes, T, A, b.h,
                                                          Act.F16_STAGED, math, h_f16=hf)
            else:
                K.stage_f16_tiles(x, b.ws, b.ws_bytes, T, A, self.E, self.d, w.gate_up.bits, b.tiled_x)
                K.linear_qw_experts_gather_grouped_swiglu(b.tiled_x, w.gate_up, self.E, b.ws, b.ws_bytes, T, A, b.h,
                                                          Act.F16_TILED, math, h_f16=hf)
        else:
            K.linear_qw_experts_gather_grouped_swiglu(x, w.gate_up, self.E, b.ws, b.ws_bytes, T, A, b.h, Act.BF16, math)
        if events is not None:
            e1.record()
            events[0].append(e0)
            events[1].append(e1)
        if before_combine is not None:
            before_combine()
        if self.ep:
            K.linear_qw_experts_combine_grouped_ep(b.h, w.down, self.E, self.E_total, self.e_lo, b.ids, b.coef, b.ws,
                                                   b.ws_bytes, b.partial, T, A, y, Act.BF16, math, out_act=out_act, h_f16=hf)
        else:
            shared = None
            if gate_logit is not None:
                shared = K.MoeSharedAdd(shared_out, gate_logit, gate_ld, self.E_total, b.router_err)
            K.linear_qw_experts_combine_grouped(b.h, w.down, self.E, b.ids, b.coef, b.ws, b.ws_bytes, b.partial, T, A, y,
                                                Act.BF16, math, shared=shared, out_act=out_act, h_f16=hf)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, y: torch.Tensor, math: Optional[MoeMath] = None):
        """x [T, d] BF16, logits [T, >= E (+1)] FP32 -> y [T, d] (BF16, or FP32 = the unrounded sums).
        With a shared expert, logits[:, E] is its gate logit and its gated output is folded into the combine."""
        T = x.shape[0]
        assert T <= self.buf.max_tokens and x.dtype == torch.bfloat16 and logits.dtype == torch.float32
        math = self.math_for(T, math)
        packed = self.route(logits, T)
        return self.run_experts(x, T, y, math, logits, packed=packed)

    def run_experts(self, x: torch.Tensor, T: int, y: torch.Tensor, math: MoeMath, logits: torch.Tensor, events=None,
                    packed: bool = False):
        """Everything after the router: shared expert, pack, routed experts, combine (+ gated shared add)."""
        if self.ep and self.w.shared_gate_up is not None:
            raise K.Error(1, "an expert-parallel rank's layer holds no shared expert: the shared expert is not sharded - run "
                             "it on the tokens' owner, outside the expert-parallel layer")
        if self.w.shared_gate_up is None:
            self.experts(x, T, y, math, events=events, packed=packed)
            return y
        b = self.buf
        sh = b.sh_y32 if y.dtype == torch.float32 else b.sh_y
        gate = logits.data_ptr() + 4 * self.E_total
        if K_is_f16(math):
            self.shared_expert(x, T, math, sh)
            self.experts(x, T, y, math, gate_logit=gate, gate_ld=logits.stride(0), shared_out=sh, events=events, packed=packed)
            return y
        # Decode: the shared expert's three small launches run on a second stream under the routed experts' weight
        # streaming (they leave most SMs idle on their own) and are joined just before the combine that adds them.
        cur = torch.cuda.current_stream()
        if b.side_stream is None:
            b.side_stream = torch.cuda.Stream(device=x.device)
            b.ev_fork, b.ev_join = torch.cuda.Event(), torch.cuda.Event()
        b.ev_fork.record(cur)
        b.side_stream.wait_event(b.ev_fork)
        with torch.cuda.stream(b.side_stream):
            self.shared_expert(x, T, math, sh)
            b.ev_join.record(b.side_stream)
        self.experts(x, T, y, math, gate_logit=gate, gate_ld=logits.stride(0), shared_out=sh, events=events,
                     before_combine=lambda: cur.wait_event(b.ev_join), packed=packed)
        return y

    def check_errors(self, what: str = "moe layer"):
        """Blocking: the reference's read_back of the error words (runtime/qwen4exp.cpp:2391-2404)."""
        K.check_router_error(self.buf.router_err, what)
        K.check_expert_error(self.buf.expert_err, what)
        K.check_grouped_status(self.buf.ws, what)
        K.check_dense_status(what)  # the shared expert's dense tcgen05 projections record here


def K_is_f16(math: MoeMath) -> bool:
    return int(math) >= int(MoeMath.WmmaF16)
