// strix_b200_shim.hpp - header-only C++ shim: the launchers of namespace strix::kernels that make up the MoE path,
// re-created over the C ABI of strix_b200.h with `hipStream_t` read as `cudaStream_t`.  With this header in place of
// kernels/moe_router.hpp, kernels/moe_grouped.hpp, kernels/linear_q4.hpp, kernels/linear_q8.hpp and
// kernels/swiglu.hpp, the call block at runtime/qwen4exp.cpp:3143-3217 (and the MTP head's at :3854-3873) compiles
// unchanged against libstrix_b200.so.  A non-zero return code is rethrown as strix::Error (strix::GpuFatalError for a
// sticky CUDA error), carrying the library's message.
//
// Inside the reference's tree the reference's own types are used (common/check.hpp, kernels/norm.hpp's Act,
// runtime/q4_device.hpp, runtime/q8_device.hpp).  Outside it (this repository's tests), layout-compatible stand-ins are
// defined here so the shim can be compiled on its own.
#pragma once

#include "strix_b200.h"

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#if __has_include("common/check.hpp") && __has_include("runtime/q4_device.hpp")
#include "common/check.hpp"
#include "kernels/norm.hpp"
#include "runtime/q4_device.hpp"
#include "runtime/q8_device.hpp"
#else
namespace strix {
class Error : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};
class GpuFatalError : public Error {
public:
    using Error::Error;
};
struct Q4DeviceView {
    const uint8_t *q = nullptr;
    const uint16_t *scale = nullptr;
    const uint16_t *minv = nullptr;
    int64_t N = 0, K = 0, G = 0;
};
struct Q8DeviceView {
    const uint8_t *q = nullptr;
    const uint16_t *scale = nullptr;
    const uint16_t *minv = nullptr;
    int64_t N = 0, K = 0, G = 0;
};
namespace kernels {
enum class Act { F32, BF16 };
}
}  // namespace strix
#endif

#ifndef STRIX_B200_NO_HIP_ALIAS
using hipStream_t = cudaStream_t;
#endif

namespace strix::kernels {

static_assert(sizeof(Q4DeviceView) == sizeof(SxbQView) && sizeof(Q8DeviceView) == sizeof(SxbQView),
              "SxbQView must keep Q4DeviceView's / Q8DeviceView's layout");

enum class MoeMath { F32, WmmaBf16, WmmaF16, WmmaF16Narrow, WmmaF16Wide, WmmaF16Wide256, WmmaF16F32Partials /* not upstream */ };
constexpr int64_t kMoeMaxExperts = 1023;
constexpr int64_t kMoeMaxSlots = 1 << 20;

struct MoeSharedAdd {
    const void *s = nullptr;
    const float *gate_logit = nullptr;
    int64_t gate_ld = 0;
    uint32_t gate_index = 0;
    uint32_t *err = nullptr;
};

namespace b200_detail {
inline void check(int rc) {
    if (rc == SXB_OK) return;
    if (rc == SXB_ERR_FATAL) throw GpuFatalError(sxb_last_error());
    throw Error(sxb_last_error());
}
template <typename View> inline const SxbQView *view(const View &w) { return reinterpret_cast<const SxbQView *>(&w); }
inline int act(Act a) { return a == Act::F32 ? SXB_ACT_F32 : SXB_ACT_BF16; }
inline SxbMoeSharedAdd shared(const MoeSharedAdd &s) { return {s.s, s.gate_logit, s.gate_ld, s.gate_index, s.err}; }
}  // namespace b200_detail

// kernels/moe_router.hpp
inline void moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                       int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, Act act, uint32_t *err,
                       hipStream_t stream) {
    b200_detail::check(sxb_moe_router(logits, ld, M, E, k, shared_logit, shared_ld, shared_id, ids, coef,
                                      b200_detail::act(act), err, stream));
}
inline void check_router_error(const uint32_t *err, const char *what) { b200_detail::check(sxb_check_router_error(err, what)); }
inline void report_router_error(const uint32_t e[3], const char *what) { b200_detail::check(sxb_report_router_error(e, what)); }
inline void moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                           uint32_t gate_index, Act act, uint32_t *err, hipStream_t stream) {
    b200_detail::check(sxb_moe_shared_add(y, s, gate_logit, gate_ld, M, N, gate_index, b200_detail::act(act), err, stream));
}
inline void moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                                  uint32_t gate_index, void *x, const float *w_in, int64_t H, Act act, uint32_t *err,
                                  hipStream_t stream) {
    b200_detail::check(sxb_moe_shared_add_inject(y, s, gate_logit, gate_ld, M, N, gate_index, x, w_in, H,
                                                 b200_detail::act(act), err, stream));
}

// kernels/hc.hpp:52-54
inline void hc_inject(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, Act act, hipStream_t stream) {
    b200_detail::check(sxb_hc_inject(x, w_in, y, T, H, d, b200_detail::act(act), stream));
}
// kernels/hc.hpp:36-50  hc_mix_down / hc_mix_up.  The chunk-major views (runtime/q4_device.hpp:37-43,
// runtime/q8_device.hpp:36-42) have the row-major views' fields; they stay separate types so that a kernel cannot be handed
// the wrong layout.
struct Q4ChunkMajorView {
    const uint8_t *q;
    const uint16_t *scale, *minv;
    int64_t N, K, G;
};
struct Q8ChunkMajorView {
    const uint8_t *q;
    const uint16_t *scale, *minv;
    int64_t N, K, G;
};
inline void hc_mix_down(const void *x, const Q4DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps,
                        float *h, float *w_in, float *inv, Act act, hipStream_t stream) {
    b200_detail::check(sxb_hc_mix_down_q4(x, reinterpret_cast<const SxbQView *>(&w), T, H, d, r, inject ? 1 : 0, eps, h, w_in, inv,
                                          b200_detail::act(act), stream));
}
inline void hc_mix_down(const void *x, const Q8DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps,
                        float *h, float *w_in, float *inv, Act act, hipStream_t stream) {
    b200_detail::check(sxb_hc_mix_down_q8(x, reinterpret_cast<const SxbQView *>(&w), T, H, d, r, inject ? 1 : 0, eps, h, w_in, inv,
                                          b200_detail::act(act), stream));
}
inline void hc_mix_up(const float *h, const Q4ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T,
                      int64_t H, int64_t d, void *u, Act act, hipStream_t stream) {
    static_assert(sizeof(Q4ChunkMajorView) == sizeof(SxbQView), "view layouts");
    b200_detail::check(sxb_hc_mix_up_q4(h, reinterpret_cast<const SxbQView *>(&w_up), x, norm_w, inv, T, H, d, u, b200_detail::act(act), stream));
}
inline void hc_mix_up(const float *h, const Q8ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T,
                      int64_t H, int64_t d, void *u, Act act, hipStream_t stream) {
    static_assert(sizeof(Q8ChunkMajorView) == sizeof(SxbQView), "view layouts");
    b200_detail::check(sxb_hc_mix_up_q8(h, reinterpret_cast<const SxbQView *>(&w_up), x, norm_w, inv, T, H, d, u, b200_detail::act(act), stream));
}

// kernels/hc_wmma.hpp:29-49, the mixes for multi-token forwards.  Two differences from the reference's declarations, both
// about scratch memory: hc_wmma_workspace_bytes also needs d, the code width and the group size (the workspace holds the
// restacked weight and the F16 operand besides the FP32 partials), and hc_mix_up_wmma takes a workspace of its own
// (hc_up_wmma_workspace_bytes) where the reference's launcher needs none.  `ws` is a void pointer, 256-byte aligned.
inline size_t hc_wmma_workspace_bytes(int64_t T, int64_t H, int64_t R, int64_t d, int bits, int64_t G) {
    const size_t n = sxb_hc_mix_down_wmma_workspace_bytes(T, H, d, R, bits, G);
    if (n == 0) throw Error(sxb_last_error());
    return n;
}
inline size_t hc_up_wmma_workspace_bytes(int64_t T, int64_t H, int64_t d, int64_t r, int bits, int64_t G) {
    const size_t n = sxb_hc_mix_up_wmma_workspace_bytes(T, H, d, r, bits, G);
    if (n == 0) throw Error(sxb_last_error());
    return n;
}
inline void hc_mix_down_wmma(const void *x, const Q4DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps,
                             float *h, float *w_in, float *inv, void *ws, size_t ws_bytes, Act act, hipStream_t stream,
                             bool inv_ready = false) {
    b200_detail::check(sxb_hc_mix_down_wmma_q4(x, reinterpret_cast<const SxbQView *>(&w), T, H, d, r, inject ? 1 : 0, eps, h, w_in, inv, ws,
                                               ws_bytes, b200_detail::act(act), inv_ready ? 1 : 0, stream));
}
inline void hc_mix_down_wmma(const void *x, const Q8DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps,
                             float *h, float *w_in, float *inv, void *ws, size_t ws_bytes, Act act, hipStream_t stream,
                             bool inv_ready = false) {
    b200_detail::check(sxb_hc_mix_down_wmma_q8(x, reinterpret_cast<const SxbQView *>(&w), T, H, d, r, inject ? 1 : 0, eps, h, w_in, inv, ws,
                                               ws_bytes, b200_detail::act(act), inv_ready ? 1 : 0, stream));
}
inline void hc_inject_inv(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, float eps, float *inv, Act act,
                          hipStream_t stream) {
    b200_detail::check(sxb_hc_inject_inv(x, w_in, y, T, H, d, eps, inv, b200_detail::act(act), stream));
}
inline void hc_mix_up_wmma(const float *h, const Q4ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T,
                           int64_t H, int64_t d, void *u, void *ws, size_t ws_bytes, Act act, hipStream_t stream) {
    b200_detail::check(sxb_hc_mix_up_wmma_q4(h, reinterpret_cast<const SxbQView *>(&w_up), x, norm_w, inv, T, H, d, u, ws, ws_bytes,
                                             b200_detail::act(act), stream));
}
inline void hc_mix_up_wmma(const float *h, const Q8ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T,
                           int64_t H, int64_t d, void *u, void *ws, size_t ws_bytes, Act act, hipStream_t stream) {
    b200_detail::check(sxb_hc_mix_up_wmma_q8(h, reinterpret_cast<const SxbQView *>(&w_up), x, norm_w, inv, T, H, d, u, ws, ws_bytes,
                                             b200_detail::act(act), stream));
}

// kernels/moe_grouped.hpp
inline size_t moe_route_workspace_bytes(int64_t M, int64_t A, int64_t E) {
    const size_t n = sxb_moe_route_workspace_bytes(M, A, E);
    if (n == 0) throw Error(sxb_last_error());
    return n;
}
inline void moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, void *ws, size_t ws_bytes, uint32_t *err,
                             hipStream_t stream) {
    b200_detail::check(sxb_moe_group_routes(ids, M, A, E, ws, ws_bytes, err, stream));
}
inline void linear_q4_experts_gather_grouped(const void *x, const Q4DeviceView &w, int64_t E, const void *ws, size_t ws_bytes,
                                             int64_t M, int64_t A, void *y, Act act, MoeMath math, hipStream_t stream) {
    b200_detail::check(sxb_linear_q4_experts_gather_grouped(x, b200_detail::view(w), E, ws, ws_bytes, M, A, y,
                                                            b200_detail::act(act), (int)math, stream));
}
inline void linear_q4_experts_gather_grouped_swiglu(const void *x, const Q4DeviceView &w, int64_t E, const void *ws,
                                                    size_t ws_bytes, int64_t M, int64_t A, void *h, Act act, MoeMath math,
                                                    hipStream_t stream, bool h_f16 = false) {
    b200_detail::check(sxb_linear_q4_experts_gather_grouped_swiglu(x, b200_detail::view(w), E, ws, ws_bytes, M, A, h,
                                                                   b200_detail::act(act), (int)math, stream, h_f16));
}
inline void linear_q4_experts_combine_grouped(const void *h, const Q4DeviceView &w, int64_t E, const int32_t *ids,
                                              const float *coef, const void *ws, size_t ws_bytes, float *partial, int64_t M,
                                              int64_t A, void *y, Act act, MoeMath math, hipStream_t stream,
                                              const MoeSharedAdd *shared = nullptr, bool h_f16 = false) {
    SxbMoeSharedAdd sh{};
    if (shared) sh = b200_detail::shared(*shared);
    b200_detail::check(sxb_linear_q4_experts_combine_grouped(h, b200_detail::view(w), E, ids, coef, ws, ws_bytes, partial, M,
                                                             A, y, b200_detail::act(act), b200_detail::act(act), (int)math,
                                                             stream, shared ? &sh : nullptr, h_f16));
}
// Q8 experts: no counterpart in the reference (its experts are Q4 / Q5); same calls on a Q8DeviceView.
inline void linear_q8_experts_gather_grouped_swiglu(const void *x, const Q8DeviceView &w, int64_t E, const void *ws,
                                                    size_t ws_bytes, int64_t M, int64_t A, void *h, Act act, MoeMath math,
                                                    hipStream_t stream, bool h_f16 = false) {
    b200_detail::check(sxb_linear_q8_experts_gather_grouped_swiglu(x, b200_detail::view(w), E, ws, ws_bytes, M, A, h,
                                                                   b200_detail::act(act), (int)math, stream, h_f16));
}
inline void linear_q8_experts_combine_grouped(const void *h, const Q8DeviceView &w, int64_t E, const int32_t *ids,
                                              const float *coef, const void *ws, size_t ws_bytes, float *partial, int64_t M,
                                              int64_t A, void *y, Act act, MoeMath math, hipStream_t stream,
                                              const MoeSharedAdd *shared = nullptr, bool h_f16 = false) {
    SxbMoeSharedAdd sh{};
    if (shared) sh = b200_detail::shared(*shared);
    b200_detail::check(sxb_linear_q8_experts_combine_grouped(h, b200_detail::view(w), E, ids, coef, ws, ws_bytes, partial, M,
                                                             A, y, b200_detail::act(act), b200_detail::act(act), (int)math,
                                                             stream, shared ? &sh : nullptr, h_f16));
}

// kernels/linear_q4.hpp, kernels/linear_q8.hpp
inline void linear_q4(const void *x, const Q4DeviceView &w, void *y, int64_t M, Act act, Act out_act, hipStream_t stream) {
    b200_detail::check(sxb_linear_q4(x, b200_detail::view(w), y, M, b200_detail::act(act), b200_detail::act(out_act), stream));
}
inline void linear_q4(const void *x, const Q4DeviceView &w, void *y, int64_t M, Act act, hipStream_t stream) {
    linear_q4(x, w, y, M, act, act, stream);
}
inline void linear_q8(const void *x, const Q8DeviceView &w, void *y, int64_t M, Act act, Act out_act, hipStream_t stream) {
    b200_detail::check(sxb_linear_q8(x, b200_detail::view(w), y, M, b200_detail::act(act), b200_detail::act(out_act), stream));
}
inline void linear_q8(const void *x, const Q8DeviceView &w, void *y, int64_t M, Act act, hipStream_t stream) {
    linear_q8(x, w, y, M, act, act, stream);
}
inline void linear_q4_experts_gather(const void *x, const Q4DeviceView &w, int64_t E, const int32_t *ids, int64_t M, int64_t A,
                                     void *y, Act act, uint32_t *err, hipStream_t stream) {
    b200_detail::check(sxb_linear_q4_experts_gather(x, b200_detail::view(w), E, ids, M, A, y, b200_detail::act(act), err, stream));
}
inline void linear_q4_experts_gather_swiglu(const void *x, const Q4DeviceView &w, int64_t E, const int32_t *ids, int64_t M,
                                            int64_t A, void *h, Act act, uint32_t *err, hipStream_t stream) {
    b200_detail::check(sxb_linear_q4_experts_gather_swiglu(x, b200_detail::view(w), E, ids, M, A, h, b200_detail::act(act), err,
                                                           stream));
}
inline void linear_q4_experts_combine(const void *h, const Q4DeviceView &w, int64_t E, const int32_t *ids, const float *coef,
                                      int64_t M, int64_t A, void *y, Act act, uint32_t *err, hipStream_t stream) {
    b200_detail::check(sxb_linear_q4_experts_combine(h, b200_detail::view(w), E, ids, coef, M, A, y, b200_detail::act(act),
                                                     b200_detail::act(act), err, stream));
}
inline void check_expert_error(const uint32_t *err, const char *what) { b200_detail::check(sxb_check_expert_error(err, what)); }
inline void report_expert_error(const uint32_t e[3], const char *what) { b200_detail::check(sxb_report_expert_error(e, what)); }

// kernels/linear_wmma.hpp: the multi-token projections on the tensor cores
inline void linear_q4_wmma(const void *x, const Q4DeviceView &w, void *y, int64_t M, Act act, Act out_act, hipStream_t stream) {
    b200_detail::check(sxb_linear_q4_wmma(x, b200_detail::view(w), y, M, b200_detail::act(act), b200_detail::act(out_act), stream));
}
inline void linear_q8_wmma(const void *x, const Q8DeviceView &w, void *y, int64_t M, Act act, Act out_act, hipStream_t stream) {
    b200_detail::check(sxb_linear_q8_wmma(x, b200_detail::view(w), y, M, b200_detail::act(act), b200_detail::act(out_act), stream));
}
// kernels/linear.hpp: BF16-weight projections (the router logits: BF16 x -> F32 y)
inline void linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, Act act, Act out_act,
                         hipStream_t stream) {
    b200_detail::check(sxb_linear_bf16w(x, w, y, M, N, K, b200_detail::act(act), b200_detail::act(out_act), stream));
}
inline void linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, Act act, hipStream_t stream) {
    linear_bf16w(x, w, y, M, N, K, act, act, stream);
}
// kernels/linear_wmma.hpp:29-30 - here for the router's dtype pair (BF16 x -> F32 y): a BF16 weight is its own single plane
inline void linear_bf16w_wmma(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, Act act, Act out_act,
                              hipStream_t stream) {
    if (act != Act::BF16 || out_act != Act::F32) throw Error("linear_bf16w_wmma: BF16 x -> F32 y only");
    b200_detail::check(sxb_router_logits_wmma(x, w, 1, nullptr, M, N, K, static_cast<float *>(y), N, stream));
}

// kernels/swiglu.hpp
inline void swiglu(const void *gu, void *h, int64_t rows, int64_t I, Act act, hipStream_t stream) {
    b200_detail::check(sxb_swiglu(gu, h, rows, I, b200_detail::act(act), stream));
}

// No counterpart upstream: the whole block (the call sequence of runtime/qwen4exp.cpp:3143-3217) as one call.
inline void moe_layer(const SxbMoeLayerArgs &args, hipStream_t stream) { b200_detail::check(sxb_moe_layer(&args, stream)); }

}  // namespace strix::kernels
