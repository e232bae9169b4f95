"""numpy front end of the CPU oracle (oracle/liboracle.so) and of the reference's own quantizers
(oracle/_ref/libstrix_ref_quant.so, compiled from the reference checkout by oracle/Makefile).

TEST INFRASTRUCTURE: the checker, never the thing measured or shipped.  BF16 data is numpy uint16 (raw bits).
"""
from __future__ import annotations

import ctypes as C
import os
import pathlib
import subprocess
from dataclasses import dataclass
from typing import Optional

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
ORACLE_SO = HERE / "liboracle.so"
REF_SO = HERE / "_ref" / "libstrix_ref_quant.so"

i64, vp = C.c_int64, C.c_void_p
F32, BF16 = 0, 1


def reference_checkout() -> Optional[str]:
    """Where the reference's sources lie on this machine: $STRIX_REFERENCE_DIR, else a `reference` directory beside the
    repository; None when neither holds formats/q4.cpp (the GPU hosts: only the prebuilt library travels there)."""
    for cand in (os.environ.get("STRIX_REFERENCE_DIR"), str(HERE.parent.parent / "reference")):
        if cand and pathlib.Path(cand, "formats", "q4.cpp").exists():
            return cand
    return None


def build(reference: Optional[str] = "") -> None:
    """Compiles the oracle, and the reference quantizers when a reference checkout is found ("" = look for one,
    None = do not)."""
    subprocess.run(["make", "-C", str(HERE), "all"], check=True, capture_output=True)
    if reference == "":
        reference = reference_checkout()
    if reference and pathlib.Path(reference, "formats", "q4.cpp").exists():
        subprocess.run(["make", "-C", str(HERE), "ref", f"REF={reference}"], check=True, capture_output=True)


_orc = None
_ref = None


def lib() -> C.CDLL:
    global _orc
    if _orc is None:
        if not ORACLE_SO.exists():
            build(None)
        _orc = C.CDLL(str(ORACLE_SO))
        _orc.orc_hardware_threads.restype = C.c_int
    return _orc


def ref_lib() -> Optional[C.CDLL]:
    """The reference's compiled quantizers, or None when they were never built on this machine."""
    global _ref
    if _ref is None and REF_SO.exists():
        _ref = C.CDLL(str(REF_SO))
    return _ref


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(vp)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, NaN / Inf preserved (common/bf16.hpp:21-27)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    special = (u & 0x7F800000) == 0x7F800000
    rounded = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    spec = ((u >> 16) | np.where(u & 0x007FFFFF, 0x0040, 0)).astype(np.uint16)
    return np.where(special, spec, rounded)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


@dataclass
class QWeight:
    """formats/q4.hpp:15-24 Q4Weight / formats/q8.hpp:19-27 Q8Weight on the host."""

    q: np.ndarray      # uint8 [N, K/2] or [N, K]
    scale: np.ndarray  # uint16 [N, K/G]
    minv: np.ndarray   # uint16 [N, K/G]
    N: int
    K: int
    G: int
    bits: int

    def rows(self, lo: int, hi: int) -> "QWeight":
        return QWeight(self.q[lo:hi], self.scale[lo:hi], self.minv[lo:hi], hi - lo, self.K, self.G, self.bits)

    def bytes(self) -> int:
        return self.q.size + 2 * self.scale.size + 2 * self.minv.size


def _quantize_with(fn, w: np.ndarray, G: int, bits: int) -> QWeight:
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    q = np.zeros((N, K // 2 if bits == 4 else K), dtype=np.uint8)
    scale = np.zeros((N, K // G), dtype=np.uint16)
    minv = np.zeros((N, K // G), dtype=np.uint16)
    rc = fn(_p(w), i64(N), i64(K), i64(G), C.c_int(bits), _p(q), _p(scale), _p(minv))
    if rc != 0:
        raise ValueError("quantize: bad shape or non-finite input")
    return QWeight(q, scale, minv, N, K, G, bits)


def quantize(w: np.ndarray, G: int, bits: int) -> QWeight:
    """The oracle's restatement of quantize_q4 / quantize_q8."""
    return _quantize_with(lib().orc_quantize, w, G, bits)


def ref_quantize(w: np.ndarray, G: int, bits: int) -> QWeight:
    """The reference's own quantize_q4 / quantize_q8 (compiled from its sources)."""
    return _quantize_with(ref_lib().ref_quantize, w, G, bits)


def dequantize(w: QWeight) -> np.ndarray:
    out = np.empty((w.N, w.K), dtype=np.float32)
    lib().orc_dequantize(_p(np.ascontiguousarray(w.q)), _p(np.ascontiguousarray(w.scale)),
                         _p(np.ascontiguousarray(w.minv)), i64(w.N), i64(w.K), i64(w.G), C.c_int(w.bits), _p(out))
    return out


def ref_dequantize(w: QWeight) -> np.ndarray:
    out = np.empty((w.N, w.K), dtype=np.float32)
    rc = ref_lib().ref_dequantize(_p(np.ascontiguousarray(w.q)), _p(np.ascontiguousarray(w.scale)),
                                  _p(np.ascontiguousarray(w.minv)), i64(w.N), i64(w.K), i64(w.G), C.c_int(w.bits),
                                  _p(out))
    if rc != 0:
        raise ValueError("ref_dequantize: the reference rejected the arrays")
    return out


def _act_of(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.uint16:
        return BF16
    raise TypeError(f"activations must be float32 or uint16 (BF16 bits), got {a.dtype}")


def moe_router(logits: np.ndarray, E: int, k: int, shared_logit: Optional[np.ndarray] = None, shared_ld: int = 1,
               shared_id: int = 0, err: Optional[np.ndarray] = None):
    """logits [M, ld >= E] float32 or BF16 bits -> ids [M, A] int32, coef [M, A] float32."""
    logits = np.ascontiguousarray(logits)
    M, ld = logits.shape
    A = k + (shared_logit is not None)
    ids = np.zeros((M, A), dtype=np.int32)
    coef = np.zeros((M, A), dtype=np.float32)
    lib().orc_moe_router(_p(logits), i64(ld), i64(M), i64(E), i64(k), _p(shared_logit), i64(shared_ld),
                         C.c_int32(shared_id), _p(ids), _p(coef), C.c_int(_act_of(logits)), _p(err))
    return ids, coef


def moe_group_routes(ids: np.ndarray, E: int, err: Optional[np.ndarray] = None):
    """ids [M, A] -> offsets [E + 2], slots [M * A] (stable counting sort, bucket E = invalid ids)."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    M, A = ids.shape
    offsets = np.zeros(E + 2, dtype=np.int32)
    slots = np.zeros(M * A, dtype=np.int32)
    lib().orc_moe_group_routes(_p(ids), i64(M), i64(A), i64(E), _p(offsets), _p(slots), _p(err))
    return offsets, slots


def linear_q(x: np.ndarray, w: QWeight, out_act: Optional[int] = None, threads: int = 0, w_f16: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x)
    M = x.shape[0]
    act = _act_of(x)
    out_act = act if out_act is None else out_act
    y = np.empty((M, w.N), dtype=np.float32 if out_act == F32 else np.uint16)
    lib().orc_linear_q(_p(x), C.c_int(act), _p(np.ascontiguousarray(w.q)), _p(np.ascontiguousarray(w.scale)),
                       _p(np.ascontiguousarray(w.minv)), i64(w.N), i64(w.K), i64(w.G), C.c_int(w.bits), _p(y),
                       C.c_int(out_act), i64(M), C.c_int(threads), C.c_int(int(w_f16)))
    return y


def swiglu(gu: np.ndarray) -> np.ndarray:
    gu = np.ascontiguousarray(gu)
    rows, two_i = gu.shape
    h = np.empty((rows, two_i // 2), dtype=gu.dtype)
    lib().orc_swiglu(_p(gu), _p(h), i64(rows), i64(two_i // 2), C.c_int(_act_of(gu)))
    return h


def experts_gather(x: np.ndarray, w: QWeight, E: int, ids: np.ndarray, swiglu_mode: int = 0,
                   err: Optional[np.ndarray] = None, threads: int = 0, w_f16: bool = False, x_f16: int = 0) -> np.ndarray:
    """swiglu_mode 0: y [M, A, N]; 1: h [M, A, N/2] with the decode rounding points; 2: one rounding (grouped F16).
    w_f16: weights as the matrix-unit path's F16 operand, f16(code * f16(scale) + f16(min)).
    x_f16: activations staged as F16: 0 kept as they are, 1 to nearest, 2 toward zero (the reference's staging)."""
    x = np.ascontiguousarray(x)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    M, A = ids.shape
    N = w.N // E
    cols = N // 2 if swiglu_mode else N
    y = np.empty((M, A, cols), dtype=x.dtype)
    lib().orc_experts_gather(_p(x), C.c_int(_act_of(x)), _p(np.ascontiguousarray(w.q)),
                             _p(np.ascontiguousarray(w.scale)), _p(np.ascontiguousarray(w.minv)), i64(w.N), i64(w.K),
                             i64(w.G), C.c_int(w.bits), i64(E), _p(ids), i64(M), i64(A), _p(y), C.c_int(swiglu_mode),
                             _p(err), C.c_int(threads), C.c_int(int(w_f16)), C.c_int(int(x_f16)))
    return y


def experts_combine(h: np.ndarray, w: QWeight, E: int, ids: np.ndarray, coef: np.ndarray, out_act: Optional[int] = None,
                    err: Optional[np.ndarray] = None, threads: int = 0, want_partial: bool = False, w_f16: bool = False,
                    x_f16: int = 0, partial_bf16: bool = False):
    """h [M, A, K] -> y [M, N] (and the per-slot dots [M*A, N] FP32 when asked).  partial_bf16: the per-slot dots are
    rounded to BF16 before the weighted sum (the reference's matrix-unit path, kernels/moe_grouped.hip:47-57)."""
    h = np.ascontiguousarray(h)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    coef = np.ascontiguousarray(coef, dtype=np.float32)
    M, A = ids.shape
    N = w.N // E
    act = _act_of(h)
    out_act = act if out_act is None else out_act
    y = np.empty((M, N), dtype=np.float32 if out_act == F32 else np.uint16)
    partial = np.zeros((M * A, N), dtype=np.float32) if want_partial else None
    lib().orc_experts_combine(_p(h), C.c_int(act), _p(np.ascontiguousarray(w.q)), _p(np.ascontiguousarray(w.scale)),
                              _p(np.ascontiguousarray(w.minv)), i64(w.N), i64(w.K), i64(w.G), C.c_int(w.bits), i64(E),
                              _p(ids), _p(coef), i64(M), i64(A), _p(y), C.c_int(out_act), _p(partial), _p(err),
                              C.c_int(threads), C.c_int(int(w_f16)), C.c_int(int(x_f16)), C.c_int(int(partial_bf16)))
    return (y, partial) if want_partial else y


def moe_shared_add(y: np.ndarray, s: np.ndarray, gate_logit: np.ndarray, gate_index: int,
                   err: Optional[np.ndarray] = None) -> np.ndarray:
    """Returns y + sigmoid(gate) * s in y's dtype; gate_logit [M] float32."""
    y = np.array(y, copy=True, order="C")
    s = np.ascontiguousarray(s)
    g = np.ascontiguousarray(gate_logit, dtype=np.float32)
    M, N = y.shape
    lib().orc_moe_shared_add(_p(y), _p(s), _p(g), i64(1), i64(M), i64(N), C.c_uint32(gate_index),
                             C.c_int(_act_of(y)), _p(err))
    return y


def moe_shared_add_inject(y, s, gate_logit, gate_index, x, w_in, err=None):
    y = np.array(y, copy=True, order="C")
    x = np.array(x, copy=True, order="C")
    s = np.ascontiguousarray(s)
    g = np.ascontiguousarray(gate_logit, dtype=np.float32)
    w_in = np.ascontiguousarray(w_in, dtype=np.float32)
    M, N = y.shape
    lib().orc_moe_shared_add_inject(_p(y), _p(s), _p(g), i64(1), i64(M), i64(N), C.c_uint32(gate_index), _p(x),
                                    _p(w_in), i64(w_in.shape[1]), C.c_int(_act_of(y)), _p(err))
    return y, x


def codes_of(w: QWeight) -> np.ndarray:
    """The integer codes [N, K] of a row-major weight (Q4: low nibble = even k, formats/q4.hpp:15-24)."""
    if w.bits == 8:
        return w.q.astype(np.float64)
    out = np.empty((w.N, w.K), dtype=np.float64)
    out[:, 0::2], out[:, 1::2] = (w.q & 0xF), (w.q >> 4)
    return out


def affine_weights(w: QWeight) -> np.ndarray:
    """code * scale + min in float64, NOT rounded to a dequantized value: what a row's dot with a 32-code chunk amounts to
    in the hyper-connection kernels, scale * sum(x * code) + min * sum(x) (kernels/hc.hip:117-123, 206-211)."""
    sc = np.repeat(bf16_to_f32(w.scale).astype(np.float64), w.G, axis=1)
    mn = np.repeat(bf16_to_f32(w.minv).astype(np.float64), w.G, axis=1)
    return codes_of(w) * sc + mn


def to_chunk_major(w: QWeight) -> QWeight:
    """formats/q4.hpp:41-55 / formats/q8.hpp: 32-code chunk c of row n at q[(c * N + n) * chunk bytes], group g's scale / min
    at [g * N + n].  Returned as a QWeight whose arrays hold that layout (q [K/32, N, chunk bytes], scale / min [K/G, N])."""
    cb = 16 if w.bits == 4 else 32
    q = np.ascontiguousarray(w.q.reshape(w.N, w.K // 32, cb).transpose(1, 0, 2))
    return QWeight(q, np.ascontiguousarray(w.scale.T), np.ascontiguousarray(w.minv.T), w.N, w.K, w.G, w.bits)


def ref_to_chunk_major(w: QWeight) -> QWeight:
    """The reference's own to_chunk_major (compiled from its sources)."""
    cb = 16 if w.bits == 4 else 32
    q = np.zeros((w.K // 32, w.N, cb), dtype=np.uint8)
    scale, minv = np.zeros((w.K // w.G, w.N), dtype=np.uint16), np.zeros((w.K // w.G, w.N), dtype=np.uint16)
    rc = ref_lib().ref_to_chunk_major(_p(np.ascontiguousarray(w.q)), _p(np.ascontiguousarray(w.scale)), _p(np.ascontiguousarray(w.minv)),
                                      i64(w.N), i64(w.K), i64(w.G), C.c_int(w.bits), _p(q), _p(scale), _p(minv))
    if rc != 0:
        raise ValueError("ref_to_chunk_major: the reference rejected the arrays")
    return QWeight(q, scale, minv, w.N, w.K, w.G, w.bits)


def _as_f16(v: np.ndarray) -> np.ndarray:
    """float64 values rounded once to IEEE half precision (to nearest even), back as float64."""
    with np.errstate(over="ignore"):
        return np.asarray(v, dtype=np.float64).astype(np.float16).astype(np.float64)


def hc_mix_down(x: np.ndarray, w: QWeight, H: int, d: int, r: int, inject: bool, eps: float, f16_operands: bool = False):
    """kernels/hc.hip:82-165 hc_mix_down in float64: X [T, H*d] (float32 values) -> h [T, r], w_in [T, H] or None, inv [T, H].
    a = sum_s inv_s * (W'_s . X_s) over the folded weight's rows, z = a / H, h = silu(z), w_in = 2 sigmoid(z),
    inv_s = 1 / sqrt(mean(X_s^2) + eps).
    f16_operands: the matrix-unit form's numerics (kernels/hc_wmma.hpp:3-8, kernels/hc_wmma.hip:75-134) - the products take
    x rounded once to F16 and the weights as f16(code * scale + min); inv still comes from the unrounded x."""
    X = np.asarray(x, dtype=np.float64).reshape(x.shape[0], H, d)
    W = affine_weights(w).reshape(w.N, H, d)
    inv = 1.0 / np.sqrt((X * X).mean(axis=2) + eps)            # [T, H]
    if f16_operands:
        X, W = _as_f16(X), _as_f16(W)
    per_stream = np.einsum("tsk,nsk->tns", X, W)                  # [T, R, H]
    z = (per_stream * inv[:, None, :]).sum(axis=2) / H
    sig = 1.0 / (1.0 + np.exp(-z))
    return z[:, :r] * sig[:, :r], (2.0 * sig[:, r:r + H] if inject else None), inv


def hc_mix_up(h: np.ndarray, w_up: QWeight, x: np.ndarray, norm_w: np.ndarray, inv: np.ndarray, H: int, d: int,
              f16_operands: bool = False) -> np.ndarray:
    """kernels/hc.hip:176-243 hc_mix_up in float64 (w_up ROW-major [H*d, r]): u [T, d], not yet rounded to the activation dtype.
    f16_operands: the matrix-unit form (kernels/hc_wmma.hip:203-272) - h rounded once to F16, weights f16(code * scale + min)."""
    T = h.shape[0]
    hh, ww = np.asarray(h, dtype=np.float64), affine_weights(w_up)
    if f16_operands:
        hh, ww = _as_f16(hh), _as_f16(ww)
    logits = hh @ ww.T                                                    # [T, H*d]
    z = 1.0 / (1.0 + np.exp(-logits))
    n = np.asarray(x, dtype=np.float64) * np.repeat(np.asarray(inv, dtype=np.float64), d, axis=1) * (1.0 + np.asarray(norm_w, dtype=np.float64))[None, :]
    return (z * n).reshape(T, H, d).sum(axis=1) / H


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())


@dataclass
class LayerWeights:
    gate_up: QWeight                  # [E * 2I, d]
    down: QWeight                     # [E * d, I]
    shared_gate_up: Optional[QWeight] = None  # [2I, d]
    shared_down: Optional[QWeight] = None     # [d, I]


def moe_layer(x: np.ndarray, logits: np.ndarray, w: LayerWeights, E: int, k: int, semantics: str = "decode",
              threads: int = 0):
    """One MoE sublayer as the reference's forward composes it (runtime/qwen4exp.cpp:3143-3217), shared expert
    separate.  x [T, d] BF16 bits, logits [T, E + 1] float32 (column E = the shared gate).
    semantics "decode": the per-slot / vector-unit kernels' numerics - FP32 dequantized weights, g and u rounded as
        stored, h = bf16(bf16(silu(g)) * u) (kernels/linear_q4.hip:268-274);
    semantics "grouped": the matrix-unit path's numerics served from 6 tokens up - activations staged as F16 toward
        zero (kernels/moe_grouped.hip:29-32), weights as F16 operands f16(code * scale + min), h = bf16(silu(g) * u)
        from the unrounded accumulators (kernels/moe_grouped.hpp:29-38, kernels/moe_grouped.hip:508-524), every
        per-slot dot of the down projection rounded to BF16 before the weighted sum (kernels/moe_grouped.hip:47-57);
    semantics "grouped_f32_partials": the same with the activations staged to nearest and the per-slot dots kept in
        FP32 - a variant kept to measure what the BF16 partials cost.
    Returns dict(ids, coef, h, y_routed_f32, y_f32, y_bf16)."""
    if semantics not in ("decode", "grouped", "grouped_f32_partials"):
        raise ValueError(f"unknown semantics {semantics!r}")
    ids, coef = moe_router(logits, E, k)
    f16 = semantics != "decode"
    xm = 0 if not f16 else (2 if semantics == "grouped" else 1)
    pb = semantics == "grouped"
    h = experts_gather(x, w.gate_up, E, ids, swiglu_mode=2 if f16 else 1, threads=threads, w_f16=f16, x_f16=xm)
    y_routed = experts_combine(h, w.down, E, ids, coef, out_act=F32, threads=threads, w_f16=f16, x_f16=xm, partial_bf16=pb)
    out = dict(ids=ids, coef=coef, h=h, y_routed_f32=y_routed)
    if w.shared_gate_up is not None:
        if f16:  # the shared expert through the same matrix-unit numerics as a dense projection (linear_q8_wmma)
            zero = np.zeros((x.shape[0], 1), dtype=np.int32)
            hs = experts_gather(x, w.shared_gate_up, 1, zero, swiglu_mode=2, threads=threads, w_f16=True, x_f16=xm)[:, 0]
        else:
            hs = swiglu(linear_q(x, w.shared_gate_up, threads=threads))
        s = linear_q(hs, w.shared_down, threads=threads, w_f16=f16)
        gate = np.ascontiguousarray(logits[:, E], dtype=np.float32)
        s32 = linear_q(hs, w.shared_down, out_act=F32, threads=threads, w_f16=f16)
        out["shared_s"], out["shared_s_f32"] = s, s32
        # FP32 view: nothing after h is rounded except what the path itself rounds (the BF16 per-slot dots of
        # "grouped") - the routed sum and the shared expert's output stay FP32, so the comparison is not at the mercy
        # of one BF16 rounding of s or y falling the other way (one such flip of an s near 1 is 4e-3, the size of the
        # whole tolerance).  BF16 view: the reference's roundings of s, y, y + g s.
        out["y_f32"] = moe_shared_add(y_routed, s32, gate, E)
        out["y_bf16"] = moe_shared_add(f32_to_bf16(y_routed), s, gate, E)
    else:
        out["y_f32"] = y_routed
        out["y_bf16"] = f32_to_bf16(y_routed)
    return out
