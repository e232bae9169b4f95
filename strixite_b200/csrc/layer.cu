// sxb_moe_layer: the call sequence of one MoE block as ONE entry point - what runtime/qwen4exp.cpp:3143-3217 issues
// launcher by launcher: router top-k, grouping of the slots by expert, gate/up + SwiGLU, down + weighted combine, and the
// always-on shared expert folded into the combine.  Everything goes to the caller's stream through the library's own
// entry points; nothing is allocated, nothing synchronizes.

#include "experts.cuh"

namespace sxb {
namespace {

int linear_dense(int bits, const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t st) {
    return bits == 4 ? sxb_linear_q4(x, w, y, M, act, out_act, st) : sxb_linear_q8(x, w, y, M, act, out_act, st);
}
int gather_swiglu(int bits, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes, int64_t M, int64_t A,
                  void *h, int act, int math, sxb_stream_t st, int h_f16) {
    return bits == 4 ? sxb_linear_q4_experts_gather_grouped_swiglu(x, w, E, ws, ws_bytes, M, A, h, act, math, st, h_f16)
                     : sxb_linear_q8_experts_gather_grouped_swiglu(x, w, E, ws, ws_bytes, M, A, h, act, math, st, h_f16);
}
int combine(int bits, const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef, const void *ws,
            size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int out_act, int math, sxb_stream_t st,
            const SxbMoeSharedAdd *shared, int h_f16) {
    return bits == 4 ? sxb_linear_q4_experts_combine_grouped(h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, SXB_ACT_BF16,
                                                             out_act, math, st, shared, h_f16)
                     : sxb_linear_q8_experts_combine_grouped(h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, SXB_ACT_BF16,
                                                             out_act, math, st, shared, h_f16);
}
int combine_ep(int bits, const void *h, const SxbQView *w, int64_t E, int64_t E_total, int64_t e_lo, const int32_t *ids,
               const float *coef, const void *ws, size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int out_act,
               int math, sxb_stream_t st, int h_f16, const PeerOut *peer) {
    const char *fn = "moe_layer (expert-parallel combine)";
    return bits == 4 ? combine_grouped<4>(fn, h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, SXB_ACT_BF16, out_act, math, st,
                                          nullptr, h_f16, E_total, e_lo, peer)
                     : combine_grouped<8>(fn, h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, SXB_ACT_BF16, out_act, math, st,
                                          nullptr, h_f16, E_total, e_lo, peer);
}

}  // namespace

int moe_layer_impl(const SxbMoeLayerArgs *a, sxb_stream_t stream, const PeerOut *peer) {
    const char *fn = "moe_layer";
    SXB_CHECK(a != nullptr, fn, ": null argument block");
    SXB_CHECK(a->gate_up != nullptr && a->down != nullptr, fn, ": null weight view");
    SXB_CHECK((a->gate_up_bits == 4 || a->gate_up_bits == 8) && (a->down_bits == 4 || a->down_bits == 8), fn, ": weight bits ",
              a->gate_up_bits, " / ", a->down_bits, ", expected 4 or 8");
    SXB_CHECK(a->M >= 1 && a->E >= 1 && a->A >= 1, fn, ": M = ", a->M, ", E = ", a->E, ", A = ", a->A);
    // a peer output makes even a single rank take the expert-parallel forms of the pack and the combine
    const bool ep = a->E_total != a->E || peer != nullptr;
    SXB_CHECK(a->E_total >= a->E && a->e_lo >= 0 && a->e_lo + a->E <= a->E_total, fn, ": experts [", a->e_lo, ", ", a->e_lo + a->E,
              ") of ", a->E_total);
    const bool shared = a->shared_gate_up != nullptr;
    SXB_CHECK(shared == (a->shared_down != nullptr), fn, ": the shared expert needs both of its weights");
    SXB_CHECK(!(shared && ep), fn, ": the shared expert is not sharded: run it on one rank, outside the expert-parallel call");
    SXB_CHECK(a->logits != nullptr || !shared, fn, ": the shared expert's gate is a column of the logits: logits must not be null");
    SXB_CHECK(a->x != nullptr && (a->y != nullptr || peer != nullptr) && a->ids != nullptr && a->coef != nullptr &&
                  a->ws != nullptr && a->h != nullptr && a->partial != nullptr && a->router_err != nullptr && a->expert_err != nullptr,
              fn, ": null buffer");
    SXB_CHECK(a->out_act == SXB_ACT_BF16 || a->out_act == SXB_ACT_F32, fn, ": output dtype ", a->out_act);
    const int64_t M = a->M, A = a->A, E = a->E, d = a->gate_up->K, I = a->gate_up->N / E / 2;
    SXB_CHECK(a->gate_up->N == E * 2 * I && a->down->N == E * d && a->down->K == I, fn, ": gate_up [", a->gate_up->N, ", ",
              a->gate_up->K, "] and down [", a->down->N, ", ", a->down->K, "] do not describe ", E, " experts");
    const int math = a->math >= 0 ? a->math : (M >= 256 ? SXB_MATH_WMMA_F16_F32_PARTIALS : SXB_MATH_F32);
    const bool tc = math >= SXB_MATH_WMMA_F16;
    SXB_CHECK(!tc || a->xs != nullptr, fn, ": the tcgen05 path needs the tile-blocked activation buffer xs (M * A * d F16)");
    auto st = static_cast<cudaStream_t>(stream);

    // router (kernels/moe_router.hpp:38-40): top-k of the first E_total logits; a shared expert's gate is column E_total.
    // logits == NULL: ids and coef already hold the routes (an expert-parallel rank receives them from the tokens' owners)
    // A small batch (decode) routes and packs in one launch.
    bool packed = false;
    if (a->logits != nullptr && !ep && M * A <= 2048) {
        if (int rc = sxb_moe_route_small(a->logits, a->logits_ld, M, a->E_total, A, 0, E, a->ids, a->coef, a->ws, a->ws_bytes,
                                         a->router_err, a->expert_err, stream))
            return rc;
        packed = true;
    } else if (a->logits != nullptr) {
        if (int rc = sxb_moe_router(a->logits, a->logits_ld, M, a->E_total, A, nullptr, 1, 0, a->ids, a->coef, SXB_ACT_F32,
                                    a->router_err, stream))
            return rc;
    }

    // the shared expert as dense projections (runtime/qwen4exp.cpp:3163-3168), in y's dtype
    if (shared) {
        SXB_CHECK(a->sh_h != nullptr && a->sh_y != nullptr, fn, ": null shared-expert buffer");
        if (!tc) {
            SXB_CHECK(a->sh_gu != nullptr, fn, ": null shared-expert buffer sh_gu");
            if (int rc = linear_dense(a->shared_bits, a->x, a->shared_gate_up, a->sh_gu, M, SXB_ACT_BF16, SXB_ACT_BF16, stream)) return rc;
            if (int rc = sxb_swiglu(a->sh_gu, a->sh_h, M, I, SXB_ACT_BF16, stream)) return rc;
            if (int rc = linear_dense(a->shared_bits, a->sh_h, a->shared_down, a->sh_y, M, SXB_ACT_BF16, a->out_act, stream)) return rc;
        } else {
            // dense projections on the tcgen05 kernel (kernels/linear_wmma.hip:69-113), SwiGLU fused into the first;
            // a wait that ran out is recorded in the routed experts' workspace header, like theirs
            SXB_CHECK(a->sh_xs != nullptr, fn, ": null shared-expert buffer sh_xs for the tcgen05 path");
            uint32_t *status = reinterpret_cast<uint32_t *>(a->ws) + 5;
            if (int rc = sxb_stage_f16_tiles(a->x, nullptr, 0, M, 1, 1, d, a->shared_bits, a->sh_xs, stream)) return rc;
            const int hf = a->shared_bits == 4 ? 3 : 4;
            const int of = a->out_act == SXB_ACT_F32 ? 1 : 0;
            int rc = a->shared_bits == 4
                         ? tc_dense<4>(fn, a->sh_xs, a->shared_gate_up, a->sh_h, M, 3, 2, hf, status, stream)
                         : tc_dense<8>(fn, a->sh_xs, a->shared_gate_up, a->sh_h, M, 3, 2, hf, status, stream);
            if (rc) return rc;
            rc = a->shared_bits == 4 ? tc_dense<4>(fn, a->sh_h, a->shared_down, a->sh_y, M, 3, of, 0, status, stream)
                                     : tc_dense<8>(fn, a->sh_h, a->shared_down, a->sh_y, M, 3, of, 0, status, stream);
            if (rc) return rc;
        }
    }

    // pack (kernels/moe_grouped.hpp:53-54)
    if (packed) {
    } else if (ep) {
        if (int rc = sxb_moe_group_routes_ep(a->ids, M, A, a->E_total, a->e_lo, E, a->ws, a->ws_bytes, a->expert_err, stream)) return rc;
    } else {
        if (int rc = sxb_moe_group_routes(a->ids, M, A, E, a->ws, a->ws_bytes, a->expert_err, stream)) return rc;
    }
    // gate/up + SwiGLU (kernels/moe_grouped.hpp:67-69)
    const int hf = tc ? (a->down_bits == 4 ? 3 : 4) : 0;
    if (tc) {
        if (int rc = sxb_stage_f16_tiles(a->x, a->ws, a->ws_bytes, M, A, E, d, a->gate_up_bits, a->xs, stream)) return rc;
        if (int rc = gather_swiglu(a->gate_up_bits, a->xs, a->gate_up, E, a->ws, a->ws_bytes, M, A, a->h, SXB_ACT_F16_TILED, math, stream, hf))
            return rc;
    } else {
        if (int rc = gather_swiglu(a->gate_up_bits, a->x, a->gate_up, E, a->ws, a->ws_bytes, M, A, a->h, SXB_ACT_BF16, math, stream, 0))
            return rc;
    }
    // down + combine (+ gated shared add) (kernels/moe_grouped.hpp:88-91)
    if (ep)
        return combine_ep(a->down_bits, a->h, a->down, E, a->E_total, a->e_lo, a->ids, a->coef, a->ws, a->ws_bytes, a->partial, M, A,
                          a->y, a->out_act, math, stream, hf, peer);
    SxbMoeSharedAdd sh{};
    if (shared) {
        sh.s = a->sh_y, sh.gate_logit = a->logits + a->E_total, sh.gate_ld = a->logits_ld, sh.gate_index = (uint32_t)a->E_total;
        sh.err = a->router_err;
    }
    return combine(a->down_bits, a->h, a->down, E, a->ids, a->coef, a->ws, a->ws_bytes, a->partial, M, A, a->y, a->out_act, math,
                   stream, shared ? &sh : nullptr, hf);
}

}  // namespace sxb

extern "C" int sxb_moe_layer(const SxbMoeLayerArgs *a, sxb_stream_t stream) { return sxb::moe_layer_impl(a, stream, nullptr); }
