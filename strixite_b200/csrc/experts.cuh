// Internal entry points shared between the expert translation units.
#pragma once

#include "route_pack.cuh"

namespace sxb {

// Where an expert-parallel rank's combine writes: row m of the T token rows belongs to rank m / t, and goes - as this
// rank's piece of it - to row (rank * t + m % t) of that rank's receive buffer [world][t][N], through a peer mapping
// (plain stores; the owner sums the pieces in rank order).
struct PeerOut {
    void *base[8];
    int world, rank;
    int64_t t;
    int f16;  // pieces stored as F16 instead of FP32
};

// stream_mma.cu - exact-product kernels (mma.sync on integer codes, FP32 scale / min per group).
template <int BITS>
int stream_gather_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                          int64_t M, int64_t A, void *y, int act, bool swiglu, sxb_stream_t stream);
template <int BITS>
int stream_partial_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                           int64_t M, int64_t A, float *partial, int act, sxb_stream_t stream);
template <int BITS>
int stream_combine_slots(const char *fn, const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                         const float *coef, int64_t M, int64_t A, void *y, int act, int out_act, uint32_t *err,
                         sxb_stream_t stream);
int combine_reduce(const char *fn, const float *partial, const int32_t *ids, const float *coef, int64_t M, int64_t A,
                   int64_t E_total, int64_t e_lo, int64_t E_local, int64_t N, void *y, int out_act,
                   const SxbMoeSharedAdd *shared, int s_act, bool partial_bf16, sxb_stream_t stream,
                   const PeerOut *peer = nullptr);
// grouped.cu: the grouped down projection + combine behind every public combine entry (checks, dispatch on math, reduce).
template <int BITS>
int combine_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E_view, const int32_t *ids, const float *coef,
                    const void *ws, size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act, int out_act,
                    int math, sxb_stream_t stream, const SxbMoeSharedAdd *shared, int h_f16, int64_t E_total, int64_t e_lo,
                    const PeerOut *peer = nullptr);
// layer.cu: sxb_moe_layer; with `peer` the combine's rows go to their owners' receive buffers instead of y.
int moe_layer_impl(const SxbMoeLayerArgs *a, sxb_stream_t stream, const PeerOut *peer);

// grouped_tc.cu - tcgen05 kernels (F16 operands, FP32 accumulation in tensor memory).
template <int BITS>
int tc_gather_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                      int64_t M, int64_t A, void *y, int act, bool swiglu, int h_f16, sxb_stream_t stream);
template <int BITS>
int tc_partial_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                       int64_t M, int64_t A, float *partial, int act, int h_f16, bool partial_bf16, sxb_stream_t stream);
// Dense projection on the same kernel (out_kind 0 BF16, 1 FP32, 2 fused SwiGLU; x_kind 0 BF16, 3 tile-blocked F16).
template <int BITS>
int tc_dense(const char *fn, const void *x, const SxbQView *w, void *y, int64_t M, int x_kind, int out_kind, int h_f16,
             uint32_t *status, sxb_stream_t stream);
// The up half of the hyper-connection mix on the same kernel: the stream combine is the epilogue (hc_tc.cu).
template <int BITS>
int tc_hc_up(const char *fn, const void *hs, const SxbQView *w, const void *x, const float *inv, const float *norm_w, void *u, int64_t M,
             int64_t d, bool f32, sxb_stream_t stream);
// f32act.cu - Act::F32 activations: the plain FP32 correctness path.  ids / ws both null: a dense projection.
template <int BITS>
int f32_gather(const char *fn, const void *x, const SxbQView *w, int64_t E, const int32_t *ids, const void *ws, int64_t M, int64_t A,
               void *y, bool swiglu, int row_div, uint32_t *err, sxb_stream_t stream);
template <int BITS>
int f32_combine(const char *fn, const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef, int64_t M,
                int64_t A, void *y, uint32_t *err, sxb_stream_t stream);
// route_pack.cu: SXB_ERR_DATA with the message for the status words {2, work item, role} of a wait that ran out.
int tc_status_error(const char *what, const uint32_t e[3]);

inline bool math_is_f16(int math) { return math >= SXB_MATH_WMMA_F16 && math <= SXB_MATH_WMMA_F16_F32_PARTIALS; }
inline bool math_ok(int math) { return math >= SXB_MATH_F32 && math <= SXB_MATH_WMMA_F16_F32_PARTIALS; }
// The reference's matrix-unit path stores the combine's per-slot dots as BF16 (kernels/moe_grouped.hip:47-57).
inline bool math_bf16_partials(int math) { return math >= SXB_MATH_WMMA_F16 && math <= SXB_MATH_WMMA_F16_WIDE256; }

}  // namespace sxb
