"""Host-side mirror of the reference's `strix::kernels` launchers for the MoE path, over the C ABI.

Same function names, argument order and meaning as kernels/moe_router.hpp, kernels/moe_grouped.hpp,
kernels/linear_q4.hpp, kernels/linear_q8.hpp and kernels/swiglu.hpp; a failed precondition raises `Error` (the
reference throws strix::Error) carrying the library's message.  Tensors are torch CUDA tensors used purely as device
memory: BF16 activations may be passed as torch.bfloat16 or as raw uint16/int16 bit tensors.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib


class Error(RuntimeError):
    """A failed precondition or launch; the reference's strix::Error (common/check.hpp:29-32)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class GpuFatalError(Error):
    """A sticky CUDA error: the context is gone (common/check.hpp:36-39)."""


class Act(enum.IntEnum):  # kernels/norm.hpp:20
    F32 = 0
    BF16 = 1
    F16_STAGED = 2  # not in the reference: F16 laid out by stage_f16 for a tensor-core operand
    F16_TILED = 3   # not in the reference: the tile-blocked form made by stage_f16_tiles


class MoeMath(enum.IntEnum):  # kernels/moe_grouped.hpp:39
    F32 = 0
    WmmaBf16 = 1
    WmmaF16 = 2
    WmmaF16Narrow = 3
    WmmaF16Wide = 4
    WmmaF16Wide256 = 5
    WmmaF16F32Partials = 6  # not in the reference: WmmaF16 with the combine's per-slot dots kept in FP32


LAUNCHES = 0  # kernels of this library launched through this module (the benchmark's gpu_launches)


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def _check(rc: int) -> None:
    _count()
    if rc != 0:
        msg = _lib.load().sxb_last_error().decode()
        raise (GpuFatalError if rc == 3 else Error)(rc, msg)


def _ptr(t) -> Optional[int]:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if not t.is_cuda:
        raise Error(1, "strixite_b200.kernels: tensors must live on a CUDA device (no CPU path exists)")
    return t.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream if isinstance(stream, int) else stream.cuda_stream


@dataclass
class QDeviceView:
    """A quantized matrix on the device: Q4DeviceView / Q8DeviceView (runtime/q4_device.hpp:14-19) plus its bit width."""

    q: torch.Tensor       # uint8 [N, K/2] (Q4) or [N, K] (Q8)
    scale: torch.Tensor   # BF16 bits [N, K/G]
    minv: torch.Tensor    # BF16 bits [N, K/G]
    N: int
    K: int
    G: int
    bits: int = 4

    def c(self) -> _lib.SxbQView:
        return _lib.SxbQView(self.q.data_ptr(), self.scale.data_ptr(), self.minv.data_ptr(), self.N, self.K, self.G)

    def bytes(self) -> int:
        return self.q.numel() + 2 * self.scale.numel() + 2 * self.minv.numel()

    def rows(self, lo: int, hi: int) -> "QDeviceView":
        """The view of rows [lo, hi) (e.g. one rank's experts of a stacked matrix)."""
        return QDeviceView(self.q[lo:hi], self.scale[lo:hi], self.minv[lo:hi], hi - lo, self.K, self.G, self.bits)


class QRawView:
    """A quantized matrix given by raw device pointers (e.g. a view into a loaded strixw file): the same interface as
    QDeviceView for the launchers."""

    def __init__(self, view: "_lib.SxbQView", bits: int, keepalive=None):
        self.view, self.bits, self.keepalive = view, bits, keepalive
        self.N, self.K, self.G = view.N, view.K, view.G

    def c(self) -> "_lib.SxbQView":
        return self.view

    def bytes(self) -> int:
        return self.N * self.K * self.bits // 8 + 4 * self.N * (self.K // self.G)


def _b(w: QDeviceView) -> str:
    if w.bits not in (4, 8):
        raise Error(1, f"experts have {w.bits} bits, expected 4 or 8")
    return f"q{w.bits}"


# ---- kernels/moe_router.hpp -----------------------------------------------------------------------------------

def moe_router(logits, ld, M, E, k, shared_logit, shared_ld, shared_id, ids, coef, act, err, stream=None):
    _check(_lib.load().sxb_moe_router(_ptr(logits), ld, M, E, k, _ptr(shared_logit), shared_ld, shared_id, _ptr(ids),
                                      _ptr(coef), int(act), _ptr(err), _stream(stream)))


def check_router_error(err, what: str):
    _check(_lib.load().sxb_check_router_error(_ptr(err), what.encode()))


def report_router_error(e, what: str):
    _check(_lib.load().sxb_report_router_error((C.c_uint32 * 3)(*[int(v) for v in e]), what.encode()))


def moe_shared_add(y, s, gate_logit, gate_ld, M, N, gate_index, act, err, stream=None):
    _check(_lib.load().sxb_moe_shared_add(_ptr(y), _ptr(s), _ptr(gate_logit), gate_ld, M, N, gate_index, int(act),
                                          _ptr(err), _stream(stream)))


def moe_shared_add_inject(y, s, gate_logit, gate_ld, M, N, gate_index, x, w_in, H, act, err, stream=None):
    _check(_lib.load().sxb_moe_shared_add_inject(_ptr(y), _ptr(s), _ptr(gate_logit), gate_ld, M, N, gate_index, _ptr(x),
                                                 _ptr(w_in), H, int(act), _ptr(err), _stream(stream)))


# ---- kernels/linear.hpp, kernels/linear_wmma.hpp: the router-logits projection; the residual add ----------------

def linear_bf16w(x, w, y, M, N, K, act, out_act=None, stream=None):
    _check(_lib.load().sxb_linear_bf16w(_ptr(x), _ptr(w), _ptr(y), M, N, K, int(act), int(act if out_act is None else out_act),
                                        _stream(stream)))


def _w_act(w) -> int:
    return int(Act.F32 if w.dtype == torch.float32 else Act.BF16)


def router_logits(x, w, bias, logits, stream=None):
    """logits [M, ld] FP32 = x [M, K] BF16 * w [N, K]^T (FP32 or BF16) + bias [N]: the streaming (decode) form."""
    M, K = x.shape
    N = w.shape[0]
    _check(_lib.load().sxb_router_logits(_ptr(x), _ptr(w), _w_act(w), _ptr(bias), M, N, K, _ptr(logits), logits.stride(0),
                                         _stream(stream)))


@dataclass
class RouterPlanes:
    """A router weight prepared for the tensor-core projection: `planes` BF16 planes [planes][Npad][K]."""

    data: torch.Tensor
    planes: int
    N: int
    K: int


def router_prepare(w: torch.Tensor, planes: Optional[int] = None, stream=None) -> RouterPlanes:
    """Splits w [N, K] (FP32: 3 planes carry every bit of it, 2 planes 16 bits; BF16: 1 plane) once, at load time."""
    N, K = w.shape
    if planes is None:
        planes = 3 if w.dtype == torch.float32 else 1
    nbytes = _lib.load().sxb_router_planes_bytes(N, K, planes)
    if nbytes == 0:
        _check(1)
    data = torch.empty(nbytes // 2, dtype=torch.int16, device=w.device)
    _check(_lib.load().sxb_router_prepare(_ptr(w), _w_act(w), N, K, planes, _ptr(data), _stream(stream)))
    return RouterPlanes(data, planes, N, K)


def router_logits_wmma(x, rp: RouterPlanes, bias, logits, stream=None):
    """The same projection on the tcgen05 tensor cores (prefill)."""
    M = x.shape[0]
    _check(_lib.load().sxb_router_logits_wmma(_ptr(x), _ptr(rp.data), rp.planes, _ptr(bias), M, rp.N, rp.K, _ptr(logits),
                                              logits.stride(0), _stream(stream)))


def residual_add(x, y, out, stream=None):
    """out = bf16(x + y); x, out BF16 (out may be x), y FP32 or BF16."""
    _check(_lib.load().sxb_residual_add(_ptr(x), _ptr(y), int(Act.F32 if y.dtype == torch.float32 else Act.BF16), _ptr(out),
                                        x.numel(), _stream(stream)))


def check_dense_status(what: str):
    _check(_lib.load().sxb_check_dense_status(what.encode()))


def set_wait_limit(ns: int):
    _check(_lib.load().sxb_set_wait_limit(int(ns)))


def linear_qw_wmma(x, w: QDeviceView, y, M, act, out_act=None, stream=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_wmma")
    _check(fn(_ptr(x), C.byref(w.c()), _ptr(y), M, int(act), int(Act.BF16 if out_act is None else out_act), _stream(stream)))


def linear_qw_wmma_swiglu(x, w: QDeviceView, h, M, act, h_f16=0, stream=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_wmma_swiglu")
    _check(fn(_ptr(x), C.byref(w.c()), _ptr(h), M, int(act), int(h_f16), _stream(stream)))


def hc_inject(x, w_in, y, T, H, d, act, stream=None):
    """kernels/hc.hpp:52-54: X[t, s*d + j] += w_in[t, s] * y[t, j], in place."""
    _check(_lib.load().sxb_hc_inject(_ptr(x), _ptr(w_in), _ptr(y), T, H, d, int(act), _stream(stream)))


def hc_mix_down(x, w: QDeviceView, T, H, d, r, inject, eps, h, w_in, inv, act, stream=None):
    """kernels/hc.hpp:36-42: X [T, H*d] -> h [T, r], w_in [T, H] (inject), inv [T, H]; w [r (+ H), H*d] Q4 or Q8."""
    fn = getattr(_lib.load(), f"sxb_hc_mix_down_{_b(w)}")
    _check(fn(_ptr(x), C.byref(w.c()), T, H, d, r, int(bool(inject)), C.c_float(eps), _ptr(h), _ptr(w_in), _ptr(inv), int(act),
              _stream(stream)))


def hc_mix_up(h, w_up: QDeviceView, x, norm_w, inv, T, H, d, u, act, stream=None):
    """kernels/hc.hpp:44-50: u [T, d] from h [T, r], the streams X, the hc_norm weight and inv; w_up [H*d, r] CHUNK-MAJOR."""
    fn = getattr(_lib.load(), f"sxb_hc_mix_up_{_b(w_up)}")
    _check(fn(_ptr(h), C.byref(w_up.c()), _ptr(x), _ptr(norm_w), _ptr(inv), T, H, d, _ptr(u), int(act), _stream(stream)))


def hc_wmma_workspace_bytes(T, H, d, R, bits, G) -> int:
    """kernels/hc_wmma.hpp:29-30: bytes of device workspace hc_mix_down_wmma needs for T tokens and R = r (+ H) weight rows."""
    n = _lib.load().sxb_hc_mix_down_wmma_workspace_bytes(T, H, d, R, int(bits), G)
    if n == 0:
        _check(1)
    return n


def hc_mix_down_wmma(x, w: QDeviceView, T, H, d, r, inject, eps, h, w_in, inv, ws, act, stream=None, inv_ready=False):
    """kernels/hc_wmma.hpp:34-39: hc_mix_down on the tensor cores (F16 operands, FP32 accumulation); ws: a uint8 tensor of
    hc_wmma_workspace_bytes, 256-byte aligned."""
    fn = getattr(_lib.load(), f"sxb_hc_mix_down_wmma_{_b(w)}")
    _check(fn(_ptr(x), C.byref(w.c()), T, H, d, r, int(bool(inject)), C.c_float(eps), _ptr(h), _ptr(w_in), _ptr(inv), _ptr(ws),
              ws.numel() * ws.element_size(), int(act), int(bool(inv_ready)), _stream(stream)))


def hc_inject_inv(x, w_in, y, T, H, d, eps, inv, act, stream=None):
    """kernels/hc_wmma.hpp:40-43: hc_inject and the next mix's inv [T, H] of the updated X, in one pass."""
    _check(_lib.load().sxb_hc_inject_inv(_ptr(x), _ptr(w_in), _ptr(y), T, H, d, C.c_float(eps), _ptr(inv), int(act), _stream(stream)))


def hc_mix_up_wmma_workspace_bytes(T, H, d, r, bits, G) -> int:
    n = _lib.load().sxb_hc_mix_up_wmma_workspace_bytes(T, H, d, r, int(bits), G)
    if n == 0:
        _check(1)
    return n


def hc_mix_up_wmma(h, w_up: QDeviceView, x, norm_w, inv, T, H, d, u, ws, act, stream=None):
    """kernels/hc_wmma.hpp:45-49: hc_mix_up on the tensor cores; w_up [H*d, r] CHUNK-MAJOR; ws: a uint8 tensor of
    hc_mix_up_wmma_workspace_bytes."""
    fn = getattr(_lib.load(), f"sxb_hc_mix_up_wmma_{_b(w_up)}")
    _check(fn(_ptr(h), C.byref(w_up.c()), _ptr(x), _ptr(norm_w), _ptr(inv), T, H, d, _ptr(u), _ptr(ws), ws.numel() * ws.element_size(),
              int(act), _stream(stream)))


def to_chunk_major(w: QDeviceView, stream=None) -> QDeviceView:
    """formats/q4.hpp:55 to_chunk_major on the device: a new view with the same codes, scales and mins chunk-major."""
    q, sc, mn = torch.empty_like(w.q), torch.empty_like(w.scale), torch.empty_like(w.minv)
    _check(_lib.load().sxb_to_chunk_major(C.byref(w.c()), w.bits, _ptr(q), _ptr(sc), _ptr(mn), _stream(stream)))
    return QDeviceView(q, sc, mn, w.N, w.K, w.G, w.bits)


# ---- kernels/moe_grouped.hpp ----------------------------------------------------------------------------------

def moe_route_workspace_bytes(M, A, E) -> int:
    n = _lib.load().sxb_moe_route_workspace_bytes(M, A, E)
    if n == 0:
        _check(1)
    return n


TC_TILES = (192, 256)  # tokens per work item of the tcgen05 kernel for tile-blocked activations (route_pack.cuh)


def route_layout(M, A, E) -> dict:
    out = (C.c_int64 * 8)()
    _check(_lib.load().sxb_route_layout(M, A, E, out))
    keys = ["header", "offsets", "slots", "tile8_bucket", "tile8_start", "tile128_bucket", "tile128_start", "total"]
    L = dict(zip(keys, list(out)))
    # two more tile lists close the workspace, each a count followed by bucket and start of up to S / rows + E + 2 tiles
    at = L["total"]
    for rows in reversed(TC_TILES):
        tmax = M * A // rows + E + 2
        at -= 1 + 2 * tmax
        L[f"tile{rows}_n"], L[f"tile{rows}_bucket"], L[f"tile{rows}_start"] = at, at + 1, at + 1 + tmax
    return L


def moe_group_routes(ids, M, A, E, ws, ws_bytes, err, stream=None):
    _count(2 if M * A > 2048 else 0)  # the multi-CTA pack is three launches
    _check(_lib.load().sxb_moe_group_routes(_ptr(ids), M, A, E, _ptr(ws), ws_bytes, _ptr(err), _stream(stream)))


def moe_route_small(logits, ld, M, E_total, k, e_lo, E_local, ids, coef, ws, ws_bytes, router_err, expert_err, stream=None):
    """moe_router + moe_group_routes[_ep] as one launch of one CTA (M * k <= 2048 slots)."""
    _check(_lib.load().sxb_moe_route_small(_ptr(logits), ld, M, E_total, k, e_lo, E_local, _ptr(ids), _ptr(coef), _ptr(ws),
                                           ws_bytes, _ptr(router_err), _ptr(expert_err), _stream(stream)))


def check_grouped_status(ws, what: str):
    _check(_lib.load().sxb_check_grouped_status(_ptr(ws), what.encode()))


def moe_group_routes_ep(ids, M, A, E_total, e_lo, E_local, ws, ws_bytes, err, stream=None):
    _count(2 if M * A > 2048 else 0)
    _check(_lib.load().sxb_moe_group_routes_ep(_ptr(ids), M, A, E_total, e_lo, E_local, _ptr(ws), ws_bytes, _ptr(err),
                                               _stream(stream)))


def linear_qw_experts_gather_grouped(x, w: QDeviceView, E, ws, ws_bytes, M, A, y, act, math, stream=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_gather_grouped")
    _check(fn(_ptr(x), C.byref(w.c()), E, _ptr(ws), ws_bytes, M, A, _ptr(y), int(act), int(math), _stream(stream)))


def linear_qw_experts_gather_grouped_swiglu(x, w: QDeviceView, E, ws, ws_bytes, M, A, h, act, math, stream=None,
                                            h_f16=False):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_gather_grouped_swiglu")
    _check(fn(_ptr(x), C.byref(w.c()), E, _ptr(ws), ws_bytes, M, A, _ptr(h), int(act), int(math), _stream(stream),
              int(h_f16)))


@dataclass
class MoeSharedAdd:  # kernels/moe_grouped.hpp:75-81
    s: torch.Tensor
    gate_logit: object  # tensor or raw pointer to token 0's gate logit
    gate_ld: int
    gate_index: int
    err: torch.Tensor

    def c(self) -> _lib.SxbMoeSharedAdd:
        return _lib.SxbMoeSharedAdd(_ptr(self.s), _ptr(self.gate_logit), self.gate_ld, self.gate_index, _ptr(self.err))


def linear_qw_experts_combine_grouped(h, w: QDeviceView, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math,
                                      stream=None, shared: Optional[MoeSharedAdd] = None, h_f16=False, out_act=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_combine_grouped")
    sh = C.byref(shared.c()) if shared is not None else None
    _count(1)  # the per-slot dots, then the reduce
    _check(fn(_ptr(h), C.byref(w.c()), E, _ptr(ids), _ptr(coef), _ptr(ws), ws_bytes, _ptr(partial), M, A, _ptr(y),
              int(act), int(act if out_act is None else out_act), int(math), _stream(stream), sh, int(h_f16)))


def linear_qw_experts_combine_grouped_ep(h, w: QDeviceView, E_local, E_total, e_lo, ids, coef, ws, ws_bytes, partial, M,
                                         A, y, act, math, stream=None, h_f16=False, out_act=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_combine_grouped_ep")
    _count(1)
    _check(fn(_ptr(h), C.byref(w.c()), E_local, E_total, e_lo, _ptr(ids), _ptr(coef), _ptr(ws), ws_bytes, _ptr(partial),
              M, A, _ptr(y), int(act), int(act if out_act is None else out_act), int(math), _stream(stream), int(h_f16)))


# ---- kernels/linear_q4.hpp, kernels/linear_q8.hpp, runtime/qweight.hpp -----------------------------------------

def linear_qw(x, w: QDeviceView, y, M, act, out_act=None, stream=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}")
    _check(fn(_ptr(x), C.byref(w.c()), _ptr(y), M, int(act), int(act if out_act is None else out_act), _stream(stream)))


def linear_q4(x, w, y, M, act, out_act=None, stream=None):
    linear_qw(x, w, y, M, act, out_act, stream)


linear_q8 = linear_q4


def linear_qw_experts_gather(x, w: QDeviceView, E, ids, M, A, y, act, err, stream=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_gather")
    _check(fn(_ptr(x), C.byref(w.c()), E, _ptr(ids), M, A, _ptr(y), int(act), _ptr(err), _stream(stream)))


def linear_qw_experts_gather_swiglu(x, w: QDeviceView, E, ids, M, A, h, act, err, stream=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_gather_swiglu")
    _check(fn(_ptr(x), C.byref(w.c()), E, _ptr(ids), M, A, _ptr(h), int(act), _ptr(err), _stream(stream)))


def linear_qw_experts_combine(h, w: QDeviceView, E, ids, coef, M, A, y, act, err, stream=None, out_act=None):
    fn = getattr(_lib.load(), f"sxb_linear_{_b(w)}_experts_combine")
    _check(fn(_ptr(h), C.byref(w.c()), E, _ptr(ids), _ptr(coef), M, A, _ptr(y), int(act),
              int(act if out_act is None else out_act), _ptr(err), _stream(stream)))


def check_expert_error(err, what: str):
    _check(_lib.load().sxb_check_expert_error(_ptr(err), what.encode()))


def report_expert_error(e, what: str):
    _check(_lib.load().sxb_report_expert_error((C.c_uint32 * 3)(*[int(v) for v in e]), what.encode()))


def stage_f16(x, M, K, bits, xh, stream=None):
    """x [M, K] BF16 -> xh [M, K] F16 in the k order of a `bits`-bit tensor-core weight operand."""
    _check(_lib.load().sxb_stage_f16(_ptr(x), M, K, bits, _ptr(xh), _stream(stream)))


def stage_f16_tiles(x, ws, ws_bytes, M, A, E, K, bits, xs, stream=None):
    """x [M, K] BF16 -> xs, the tile-blocked F16 operand form for the tiles of grouping workspace ws."""
    _check(_lib.load().sxb_stage_f16_tiles(_ptr(x), _ptr(ws), ws_bytes, M, A, E, K, bits, _ptr(xs), _stream(stream)))


# ---- kernels/swiglu.hpp ---------------------------------------------------------------------------------------

def swiglu(gu, h, rows, I, act, stream=None):
    _check(_lib.load().sxb_swiglu(_ptr(gu), _ptr(h), rows, I, int(act), _stream(stream)))


# ---- formats/q4.hpp, formats/q8.hpp (on the device) -----------------------------------------------------------

def quantize(w: torch.Tensor, G: int, bits: int, err: Optional[torch.Tensor] = None, stream=None) -> QDeviceView:
    """quantize_q4 / quantize_q8 (formats/q4.hpp:32, formats/q8.hpp:32) of an FP32 [N, K] tensor on the device."""
    if w.dtype != torch.float32 or w.dim() != 2 or not w.is_contiguous():
        raise Error(1, "quantize: w must be a contiguous FP32 [N, K] tensor")
    N, K = w.shape
    if bits not in (4, 8) or G not in (32, 64, 128) or K % G:
        raise Error(1, f"quantize: bits = {bits}, G = {G}, K = {K} unsupported")
    q = torch.empty((N, K // 2 if bits == 4 else K), dtype=torch.uint8, device=w.device)
    scale = torch.empty((N, K // G), dtype=torch.int16, device=w.device)
    minv = torch.empty((N, K // G), dtype=torch.int16, device=w.device)
    own = err is None
    if own:
        err = torch.zeros(4, dtype=torch.int32, device=w.device)
    _check(_lib.load().sxb_quantize(_ptr(w), N, K, G, bits, _ptr(q), _ptr(scale), _ptr(minv), _ptr(err), _stream(stream)))
    if own and int(err[0].item()) != 0:
        raise Error(1, f"quantize: non-finite weight at [{int(err[1])}, {int(err[2])}]")
    return QDeviceView(q, scale, minv, N, K, G, bits)


# ---- the whole block as one call ------------------------------------------------------------------------------

def _layer_args(x, logits, y, gate_up, down, E, A, ids, coef, ws, ws_bytes, h, partial, router_err, expert_err, xs, math, E_total,
                e_lo, shared_gate_up, shared_down, sh_gu, sh_h, sh_y, sh_xs):
    M = x.shape[0]
    gu, dn = gate_up.c(), down.c()
    a = _lib.SxbMoeLayerArgs()
    a.M, a.E, a.A, a.E_total, a.e_lo = M, E, A, (E if E_total is None else E_total), e_lo
    a.gate_up, a.down, a.gate_up_bits, a.down_bits = C.pointer(gu), C.pointer(dn), gate_up.bits, down.bits
    keep = [gu, dn]
    if shared_gate_up is not None:
        sgu, sdn = shared_gate_up.c(), shared_down.c()
        keep += [sgu, sdn]
        a.shared_gate_up, a.shared_down, a.shared_bits = C.pointer(sgu), C.pointer(sdn), shared_gate_up.bits
    a.x, a.logits, a.logits_ld, a.y = _ptr(x), _ptr(logits), (logits.stride(0) if logits is not None else 0), _ptr(y)
    a.out_act = int(Act.F32 if y.dtype == torch.float32 else Act.BF16)
    a.math = -1 if math is None else int(math)
    a.ids, a.coef, a.ws, a.ws_bytes, a.h, a.partial = _ptr(ids), _ptr(coef), _ptr(ws), ws_bytes, _ptr(h), _ptr(partial)
    a.xs = _ptr(xs) if xs is not None else None
    for name, t in (("sh_gu", sh_gu), ("sh_h", sh_h), ("sh_y", sh_y), ("sh_xs", sh_xs)):
        setattr(a, name, _ptr(t) if t is not None else None)
    a.router_err, a.expert_err = _ptr(router_err), _ptr(expert_err)
    return a, keep


def moe_layer(x, logits, y, gate_up: QDeviceView, down: QDeviceView, E, A, ids, coef, ws, ws_bytes, h, partial, router_err,
              expert_err, xs=None, math=None, E_total=None, e_lo=0, shared_gate_up: Optional[QDeviceView] = None,
              shared_down: Optional[QDeviceView] = None, sh_gu=None, sh_h=None, sh_y=None, sh_xs=None, stream=None):
    """sxb_moe_layer: router, grouping, gate/up + SwiGLU, down + combine (+ shared expert) enqueued by one C call.
    x [M, d] BF16, logits [M, ld] FP32 (None: ids / coef already hold the routes), y [M, d] BF16 or FP32; the rest are the
    caller's work buffers."""
    a, keep = _layer_args(x, logits, y, gate_up, down, E, A, ids, coef, ws, ws_bytes, h, partial, router_err, expert_err, xs, math,
                          E_total, e_lo, shared_gate_up, shared_down, sh_gu, sh_h, sh_y, sh_xs)
    _count(8)
    _check(_lib.load().sxb_moe_layer(C.byref(a), _stream(stream)))


# ---- expert parallelism over the C ABI (no counterpart in the reference) ------------------------------------------

def ep_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    _check(_lib.load().sxb_ep_unique_id(buf))
    return bytes(buf)


class EpContext:
    """A rank's expert-parallel context (sxb_ep_create): NCCL communicator, exchange buffers, peer mappings.
    return_path: 0 reduce-scatter, 1 peer stores of FP32 pieces, 2 of F16 pieces."""

    def __init__(self, unique_id: bytes, world: int, rank: int, T: int, d: int, A: int, return_path: int = 1):
        self.handle = C.c_void_p()
        idb = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        _check(_lib.load().sxb_ep_create(idb, world, rank, T, d, A, return_path, C.byref(self.handle)))
        self.world, self.rank, self.T, self.return_path = world, rank, T, return_path

    def layer(self, x_loc, logits_loc, y_loc, gate_up: QDeviceView, down: QDeviceView, E_local, E_total, e_lo, A, ids, coef, ws,
              ws_bytes, h, partial, router_err, expert_err, xs=None, math=None, stream=None):
        """sxb_moe_layer_ep on this rank's rows; ids / coef / ws / h / partial / xs are sized for all T rows."""
        a, keep = _layer_args(x_loc, logits_loc, y_loc, gate_up, down, E_local, A, ids, coef, ws, ws_bytes, h, partial, router_err,
                              expert_err, xs, math, E_total, e_lo, None, None, None, None, None, None)
        _count(9)
        _check(_lib.load().sxb_moe_layer_ep(self.handle, C.byref(a), _stream(stream)))

    def set_timing(self, on: bool):
        _check(_lib.load().sxb_ep_set_timing(self.handle, int(on)))

    def timing(self) -> dict:
        ms = (C.c_float * 5)()
        n = C.c_int()
        _check(_lib.load().sxb_ep_timing(self.handle, ms, C.byref(n)))
        names = ("route", "gather_wait", "experts", "return", "sum")
        return {"layers": n.value, **{k: float(v) for k, v in zip(names, ms)}}

    def close(self):
        if self.handle:
            _lib.load().sxb_ep_destroy(self.handle)
            self.handle = C.c_void_p()
