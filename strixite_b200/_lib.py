"""ctypes binding of libstrix_b200.so, the C ABI declared in include/strix_b200.h.

The library is the product: there is no fallback.  Importing this module without the built library raises, and so
does any call when the loaded library reports an error.
"""
from __future__ import annotations

import ctypes as C
import pathlib

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "libstrix_b200.so"

i64, i32, u32, sz, vp, cp = C.c_int64, C.c_int32, C.c_uint32, C.c_size_t, C.c_void_p, C.c_char_p


class SxbQView(C.Structure):
    """runtime/q4_device.hpp:14-19 Q4DeviceView / runtime/q8_device.hpp:13-18 Q8DeviceView."""

    _fields_ = [("q", vp), ("scale", vp), ("minv", vp), ("N", i64), ("K", i64), ("G", i64)]


class SxbMoeSharedAdd(C.Structure):
    """kernels/moe_grouped.hpp:75-81 MoeSharedAdd."""

    _fields_ = [("s", vp), ("gate_logit", vp), ("gate_ld", i64), ("gate_index", u32), ("err", vp)]


class SxbStrixwTensor(C.Structure):
    """formats/strixw.hpp:37-48 StrixwTensor, flattened (include/strix_b200.h)."""

    _fields_ = [("name", cp), ("encoding", C.c_int), ("ndim", C.c_int), ("shape", i64 * 8), ("group_size", i64), ("experts", i64),
                ("n_parts", C.c_int), ("n_components", C.c_int), ("component_role", C.c_int * 3), ("component_offset", C.c_uint64 * 3),
                ("component_bytes", C.c_uint64 * 3), ("component_hash", C.c_uint64 * 3)]


class SxbMoeLayerArgs(C.Structure):
    """The argument block of sxb_moe_layer (include/strix_b200.h), field for field."""

    _fields_ = [("M", i64), ("E", i64), ("A", i64), ("E_total", i64), ("e_lo", i64),
                ("gate_up", C.POINTER(SxbQView)), ("down", C.POINTER(SxbQView)), ("gate_up_bits", C.c_int), ("down_bits", C.c_int),
                ("shared_gate_up", C.POINTER(SxbQView)), ("shared_down", C.POINTER(SxbQView)), ("shared_bits", C.c_int),
                ("x", vp), ("logits", vp), ("logits_ld", i64), ("y", vp), ("out_act", C.c_int), ("math", C.c_int),
                ("ids", vp), ("coef", vp), ("ws", vp), ("ws_bytes", sz), ("h", vp), ("partial", vp), ("xs", vp),
                ("sh_gu", vp), ("sh_h", vp), ("sh_y", vp), ("sh_ids", vp), ("sh_coef", vp), ("sh_ws", vp), ("sh_ws_bytes", sz),
                ("sh_partial", vp), ("sh_xs", vp), ("router_err", vp), ("expert_err", vp)]


QV = C.POINTER(SxbQView)
SA = C.POINTER(SxbMoeSharedAdd)

# name -> (restype, argtypes); mirrors include/strix_b200.h declaration by declaration.
SIGNATURES = {
    "sxb_last_error": (cp, []),
    "sxb_version": (cp, []),
    "sxb_moe_router": (C.c_int, [vp, i64, i64, i64, i64, vp, i64, i32, vp, vp, C.c_int, vp, vp]),
    "sxb_check_router_error": (C.c_int, [vp, cp]),
    "sxb_report_router_error": (C.c_int, [C.POINTER(u32), cp]),
    "sxb_moe_shared_add": (C.c_int, [vp, vp, vp, i64, i64, i64, u32, C.c_int, vp, vp]),
    "sxb_moe_shared_add_inject": (C.c_int, [vp, vp, vp, i64, i64, i64, u32, vp, vp, i64, C.c_int, vp, vp]),
    "sxb_moe_route_workspace_bytes": (sz, [i64, i64, i64]),
    "sxb_moe_group_routes": (C.c_int, [vp, i64, i64, i64, vp, sz, vp, vp]),
    "sxb_moe_group_routes_ep": (C.c_int, [vp, i64, i64, i64, i64, i64, vp, sz, vp, vp]),
    "sxb_check_grouped_status": (C.c_int, [vp, cp]),
    "sxb_route_layout": (C.c_int, [i64, i64, i64, C.POINTER(i64)]),
    "sxb_linear_q4": (C.c_int, [vp, QV, vp, i64, C.c_int, C.c_int, vp]),
    "sxb_linear_q8": (C.c_int, [vp, QV, vp, i64, C.c_int, C.c_int, vp]),
    "sxb_stage_f16": (C.c_int, [vp, i64, i64, C.c_int, vp, vp]),
    "sxb_stage_f16_tiles": (C.c_int, [vp, vp, sz, i64, i64, i64, i64, C.c_int, vp, vp]),
    "sxb_swiglu": (C.c_int, [vp, vp, i64, i64, C.c_int, vp]),
    "sxb_check_expert_error": (C.c_int, [vp, cp]),
    "sxb_report_expert_error": (C.c_int, [C.POINTER(u32), cp]),
    "sxb_quantize": (C.c_int, [vp, i64, i64, i64, C.c_int, vp, vp, vp, vp, vp]),
    "sxb_moe_layer": (C.c_int, [C.POINTER(SxbMoeLayerArgs), vp]),
    "sxb_set_wait_limit": (C.c_int, [C.c_uint64]),
    "sxb_test_skip_ring_slot": (C.c_int, [C.c_int]),
    "sxb_check_dense_status": (C.c_int, [cp]),
    "sxb_linear_q4_wmma": (C.c_int, [vp, QV, vp, i64, C.c_int, C.c_int, vp]),
    "sxb_linear_q8_wmma": (C.c_int, [vp, QV, vp, i64, C.c_int, C.c_int, vp]),
    "sxb_linear_q4_wmma_swiglu": (C.c_int, [vp, QV, vp, i64, C.c_int, C.c_int, vp]),
    "sxb_linear_q8_wmma_swiglu": (C.c_int, [vp, QV, vp, i64, C.c_int, C.c_int, vp]),
    "sxb_linear_bf16w": (C.c_int, [vp, vp, vp, i64, i64, i64, C.c_int, C.c_int, vp]),
    "sxb_router_logits": (C.c_int, [vp, vp, C.c_int, vp, i64, i64, i64, vp, i64, vp]),
    "sxb_router_planes_bytes": (sz, [i64, i64, C.c_int]),
    "sxb_router_prepare": (C.c_int, [vp, C.c_int, i64, i64, C.c_int, vp, vp]),
    "sxb_router_logits_wmma": (C.c_int, [vp, vp, C.c_int, vp, i64, i64, i64, vp, i64, vp]),
    "sxb_residual_add": (C.c_int, [vp, vp, C.c_int, vp, i64, vp]),
    "sxb_ep_unique_id": (C.c_int, [vp]),
    "sxb_ep_create": (C.c_int, [vp, C.c_int, C.c_int, i64, i64, i64, C.c_int, C.POINTER(vp)]),
    "sxb_ep_destroy": (C.c_int, [vp]),
    "sxb_moe_layer_ep": (C.c_int, [vp, C.POINTER(SxbMoeLayerArgs), vp]),
    "sxb_ep_set_timing": (C.c_int, [vp, C.c_int]),
    "sxb_ep_timing": (C.c_int, [vp, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "sxb_strixw_open": (C.c_int, [cp, C.POINTER(vp)]),
    "sxb_strixw_close": (C.c_int, [vp]),
    "sxb_strixw_tensor_count": (i64, [vp]),
    "sxb_strixw_tensor": (C.c_int, [vp, i64, C.POINTER(SxbStrixwTensor)]),
    "sxb_strixw_find": (C.c_int, [vp, cp, C.POINTER(SxbStrixwTensor)]),
    "sxb_strixw_part": (C.c_int, [vp, cp, C.c_int, C.POINTER(cp), C.POINTER(i64), C.POINTER(i64)]),
    "sxb_strixw_meta": (cp, [vp, cp]),
    "sxb_strixw_data": (vp, [vp, cp, C.c_int]),
    "sxb_strixw_verify": (C.c_int, [vp, C.c_int]),
    "sxb_strix_hash64": (C.c_uint64, [vp, sz]),
    "sxb_strixw_load": (C.c_int, [vp, C.c_int, vp]),
    "sxb_strixw_load_seconds": (C.c_double, [vp]),
    "sxb_strixw_device_ptr": (vp, [vp, cp, C.c_int]),
    "sxb_strixw_qview": (C.c_int, [vp, cp, i64, i64, C.POINTER(SxbQView), C.POINTER(C.c_int)]),
    "sxb_strixw_expert_views": (C.c_int, [vp, cp, i64, C.POINTER(SxbQView), C.POINTER(SxbQView), C.POINTER(C.c_int)]),
    "sxb_hc_inject": (C.c_int, [vp, vp, vp, i64, i64, i64, C.c_int, vp]),
    "sxb_hc_mix_down_q4": (C.c_int, [vp, QV, i64, i64, i64, i64, C.c_int, C.c_float, vp, vp, vp, C.c_int, vp]),
    "sxb_hc_mix_down_q8": (C.c_int, [vp, QV, i64, i64, i64, i64, C.c_int, C.c_float, vp, vp, vp, C.c_int, vp]),
    "sxb_hc_mix_up_q4": (C.c_int, [vp, QV, vp, vp, vp, i64, i64, i64, vp, C.c_int, vp]),
    "sxb_hc_mix_up_q8": (C.c_int, [vp, QV, vp, vp, vp, i64, i64, i64, vp, C.c_int, vp]),
    "sxb_to_chunk_major": (C.c_int, [QV, C.c_int, vp, vp, vp, vp]),
    "sxb_hc_mix_down_wmma_workspace_bytes": (sz, [i64, i64, i64, i64, C.c_int, i64]),
    "sxb_hc_mix_down_wmma_q4": (C.c_int, [vp, QV, i64, i64, i64, i64, C.c_int, C.c_float, vp, vp, vp, vp, sz, C.c_int, C.c_int, vp]),
    "sxb_hc_mix_down_wmma_q8": (C.c_int, [vp, QV, i64, i64, i64, i64, C.c_int, C.c_float, vp, vp, vp, vp, sz, C.c_int, C.c_int, vp]),
    "sxb_hc_inject_inv": (C.c_int, [vp, vp, vp, i64, i64, i64, C.c_float, vp, C.c_int, vp]),
    "sxb_hc_mix_up_wmma_workspace_bytes": (sz, [i64, i64, i64, i64, C.c_int, i64]),
    "sxb_hc_mix_up_wmma_q4": (C.c_int, [vp, QV, vp, vp, vp, i64, i64, i64, vp, vp, sz, C.c_int, vp]),
    "sxb_hc_mix_up_wmma_q8": (C.c_int, [vp, QV, vp, vp, vp, i64, i64, i64, vp, vp, sz, C.c_int, vp]),
    "sxb_moe_route_small": (C.c_int, [vp, i64, i64, i64, i64, i64, i64, vp, vp, vp, sz, vp, vp, vp]),
}
for _b in ("q4", "q8"):
    SIGNATURES[f"sxb_linear_{_b}_experts_gather"] = (C.c_int, [vp, QV, i64, vp, i64, i64, vp, C.c_int, vp, vp])
    SIGNATURES[f"sxb_linear_{_b}_experts_gather_swiglu"] = (C.c_int, [vp, QV, i64, vp, i64, i64, vp, C.c_int, vp, vp])
    SIGNATURES[f"sxb_linear_{_b}_experts_combine"] = (
        C.c_int, [vp, QV, i64, vp, vp, i64, i64, vp, C.c_int, C.c_int, vp, vp])
    SIGNATURES[f"sxb_linear_{_b}_experts_gather_grouped"] = (
        C.c_int, [vp, QV, i64, vp, sz, i64, i64, vp, C.c_int, C.c_int, vp])
    SIGNATURES[f"sxb_linear_{_b}_experts_gather_grouped_swiglu"] = (
        C.c_int, [vp, QV, i64, vp, sz, i64, i64, vp, C.c_int, C.c_int, vp, C.c_int])
    SIGNATURES[f"sxb_linear_{_b}_experts_combine_grouped"] = (
        C.c_int, [vp, QV, i64, vp, vp, vp, sz, vp, i64, i64, vp, C.c_int, C.c_int, C.c_int, vp, SA, C.c_int])
    SIGNATURES[f"sxb_linear_{_b}_experts_combine_grouped_ep"] = (
        C.c_int, [vp, QV, i64, i64, i64, vp, vp, vp, sz, vp, i64, i64, vp, C.c_int, C.c_int, C.c_int, vp, C.c_int])

SIGNATURES["sxb_linear_q4_experts_combine_grouped_noalloc"] = (
    C.c_int, [vp, QV, i64, vp, vp, vp, sz, i64, i64, vp, C.c_int, C.c_int, C.c_int, vp, SA, C.c_int])

_lib = None


def load() -> C.CDLL:
    """Loads the library once; raises if it has not been built (python -m strixite_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m strixite_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
