// The grouped expert entry points (kernels/moe_grouped.hpp:58-91) and the per-slot combine
// (kernels/linear_q4.hpp:44-46): argument checks and the dispatch on MoeMath between the exact-product streaming
// kernels (stream_mma.cu) and the tcgen05 kernels (grouped_tc.cu).

#include "experts.cuh"

namespace sxb {
namespace {

template <int BITS>
int gather_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes, int64_t M,
                   int64_t A, void *y, int act, int math, bool swiglu, int h_f16, sxb_stream_t stream) {
    SXB_CHECK(math_ok(math), fn, ": unknown math ", math);
    SXB_CHECK(h_f16 >= 0 && h_f16 <= 4, fn, ": h_f16 = ", h_f16, ", expected 0..4");
    SXB_CHECK(!h_f16 || (act != SXB_ACT_F32 && math_is_f16(math)), fn,
              ": F16 h needs BF16 activations and a WMMA_F16 math, got ", act_name(act), " math ", math);
    SXB_CHECK((act != SXB_ACT_F16_STAGED && act != SXB_ACT_F16_TILED) || math_is_f16(math), fn, ": staged F16 activations need a WMMA_F16 math");
    if (math_is_f16(math) && act != SXB_ACT_F32) return tc_gather_grouped<BITS>(fn, x, w, E, ws, ws_bytes, M, A, y, act, swiglu, h_f16, stream);
    return stream_gather_grouped<BITS>(fn, x, w, E, ws, ws_bytes, M, A, y, act, swiglu, stream);
}

}  // namespace

template <int BITS>
int combine_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E_view, const int32_t *ids, const float *coef,
                    const void *ws, size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act, int out_act,
                    int math, sxb_stream_t stream, const SxbMoeSharedAdd *shared, int h_f16, int64_t E_total,
                    int64_t e_lo, const PeerOut *peer) {
    SXB_CHECK(math_ok(math), fn, ": unknown math ", math);
    SXB_CHECK(h_f16 >= 0 && h_f16 <= 4, fn, ": h_f16 = ", h_f16, ", expected 0..4");
    SXB_CHECK(!h_f16 || (act == SXB_ACT_BF16 && math_is_f16(math)), fn,
              ": F16 h needs BF16 activations and a WMMA_F16 math, got ", act_name(act), " math ", math);
    SXB_CHECK(ids != nullptr && coef != nullptr && partial != nullptr && (y != nullptr || peer != nullptr) && w != nullptr, fn,
              ": null pointer (ids=", (const void *)ids, ", coef=", (const void *)coef, ", partial=", (const void *)partial,
              ", y=", y, ")");
    SXB_CHECK(E_view >= 1 && w->N % E_view == 0, fn, ": weight has ", w->N, " rows for E = ", E_view, " experts");
    const int64_t N = w->N / E_view;
    SXB_CHECK(act_ok(out_act) && (out_act == act || out_act == SXB_ACT_F32), fn, ": output dtype ", act_name(out_act),
              " with activations ", act_name(act), " unsupported (same dtype, or F32)");
    SXB_CHECK(apart(partial, M * A * N * 4, h, M * A * w->K * act_bytes(act)), fn, ": partial overlaps h");
    SXB_CHECK(peer != nullptr || apart(y, M * N * act_bytes(out_act), h, M * A * w->K * act_bytes(act)), fn, ": y overlaps h");
    // FP32 activations take the plain FP32 path whatever the math (the F16 kinds are defined for BF16 activations)
    const bool tc = math_is_f16(math) && act != SXB_ACT_F32;
    const bool pb = tc && math_bf16_partials(math);
    int rc = tc
                 ? tc_partial_grouped<BITS>(fn, h, w, E_view, ws, ws_bytes, M, A, partial, act, h_f16, pb, stream)
                 : stream_partial_grouped<BITS>(fn, h, w, E_view, ws, ws_bytes, M, A, partial, act, stream);
    if (rc) return rc;
    return combine_reduce(fn, partial, ids, coef, M, A, E_total, e_lo, E_view, N, y, out_act, shared, out_act, pb, stream, peer);
}

template int combine_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const float *, const void *,
                                size_t, float *, int64_t, int64_t, void *, int, int, int, sxb_stream_t, const SxbMoeSharedAdd *,
                                int, int64_t, int64_t, const PeerOut *);
template int combine_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const float *, const void *,
                                size_t, float *, int64_t, int64_t, void *, int, int, int, sxb_stream_t, const SxbMoeSharedAdd *,
                                int, int64_t, int64_t, const PeerOut *);

}  // namespace sxb

using namespace sxb;

extern "C" {

int sxb_linear_q4_experts_gather_grouped(const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                                         int64_t M, int64_t A, void *y, int act, int math, sxb_stream_t stream) {
    return gather_grouped<4>("linear_q4_experts_gather_grouped", x, w, E, ws, ws_bytes, M, A, y, act, math, false, 0,
                             stream);
}
int sxb_linear_q8_experts_gather_grouped(const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                                         int64_t M, int64_t A, void *y, int act, int math, sxb_stream_t stream) {
    return gather_grouped<8>("linear_q8_experts_gather_grouped", x, w, E, ws, ws_bytes, M, A, y, act, math, false, 0,
                             stream);
}
int sxb_linear_q4_experts_gather_grouped_swiglu(const void *x, const SxbQView *w, int64_t E, const void *ws,
                                                size_t ws_bytes, int64_t M, int64_t A, void *h, int act, int math,
                                                sxb_stream_t stream, int h_f16) {
    return gather_grouped<4>("linear_q4_experts_gather_grouped_swiglu", x, w, E, ws, ws_bytes, M, A, h, act, math, true,
                             h_f16, stream);
}
int sxb_linear_q8_experts_gather_grouped_swiglu(const void *x, const SxbQView *w, int64_t E, const void *ws,
                                                size_t ws_bytes, int64_t M, int64_t A, void *h, int act, int math,
                                                sxb_stream_t stream, int h_f16) {
    return gather_grouped<8>("linear_q8_experts_gather_grouped_swiglu", x, w, E, ws, ws_bytes, M, A, h, act, math, true,
                             h_f16, stream);
}
int sxb_linear_q4_experts_combine_grouped(const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                                          const float *coef, const void *ws, size_t ws_bytes, float *partial, int64_t M,
                                          int64_t A, void *y, int act, int out_act, int math, sxb_stream_t stream,
                                          const SxbMoeSharedAdd *shared, int h_f16) {
    return combine_grouped<4>("linear_q4_experts_combine_grouped", h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act,
                              out_act, math, stream, shared, h_f16, E, 0, nullptr);
}
int sxb_linear_q8_experts_combine_grouped(const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                                          const float *coef, const void *ws, size_t ws_bytes, float *partial, int64_t M,
                                          int64_t A, void *y, int act, int out_act, int math, sxb_stream_t stream,
                                          const SxbMoeSharedAdd *shared, int h_f16) {
    return combine_grouped<8>("linear_q8_experts_combine_grouped", h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act,
                              out_act, math, stream, shared, h_f16, E, 0, nullptr);
}
int sxb_linear_q4_experts_combine_grouped_ep(const void *h, const SxbQView *w, int64_t E_local, int64_t E_total,
                                             int64_t e_lo, const int32_t *ids, const float *coef, const void *ws,
                                             size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act,
                                             int out_act, int math, sxb_stream_t stream, int h_f16) {
    SXB_CHECK(e_lo >= 0 && E_local >= 1 && e_lo + E_local <= E_total, "linear_q4_experts_combine_grouped_ep: experts [",
              e_lo, ", ", e_lo + E_local, ") outside [0, ", E_total, ")");
    return combine_grouped<4>("linear_q4_experts_combine_grouped_ep", h, w, E_local, ids, coef, ws, ws_bytes, partial, M, A,
                              y, act, out_act, math, stream, nullptr, h_f16, E_total, e_lo, nullptr);
}
int sxb_linear_q8_experts_combine_grouped_ep(const void *h, const SxbQView *w, int64_t E_local, int64_t E_total,
                                             int64_t e_lo, const int32_t *ids, const float *coef, const void *ws,
                                             size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act,
                                             int out_act, int math, sxb_stream_t stream, int h_f16) {
    SXB_CHECK(e_lo >= 0 && E_local >= 1 && e_lo + E_local <= E_total, "linear_q8_experts_combine_grouped_ep: experts [",
              e_lo, ", ", e_lo + E_local, ") outside [0, ", E_total, ")");
    return combine_grouped<8>("linear_q8_experts_combine_grouped_ep", h, w, E_local, ids, coef, ws, ws_bytes, partial, M, A,
                              y, act, out_act, math, stream, nullptr, h_f16, E_total, e_lo, nullptr);
}

int sxb_linear_q4_experts_combine(const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef,
                                  int64_t M, int64_t A, void *y, int act, int out_act, uint32_t *err, sxb_stream_t stream) {
    return stream_combine_slots<4>("linear_q4_experts_combine", h, w, E, ids, coef, M, A, y, act, out_act, err, stream);
}
int sxb_linear_q8_experts_combine(const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef,
                                  int64_t M, int64_t A, void *y, int act, int out_act, uint32_t *err, sxb_stream_t stream) {
    return stream_combine_slots<8>("linear_q8_experts_combine", h, w, E, ids, coef, M, A, y, act, out_act, err, stream);
}

}  // extern "C"
