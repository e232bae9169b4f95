// Internal entry points shared between the expert translation units.
#pragma once

#include "route_pack.cuh"

namespace sxb {

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
                   const SxbMoeSharedAdd *shared, int s_act, sxb_stream_t stream);

// grouped_tc.cu - tcgen05 kernels (F16 operands, FP32 accumulation in tensor memory).
template <int BITS>
int tc_gather_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                      int64_t M, int64_t A, void *y, int act, bool swiglu, int h_f16, sxb_stream_t stream);
template <int BITS>
int tc_partial_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                       int64_t M, int64_t A, float *partial, int act, int h_f16, sxb_stream_t stream);

inline bool math_is_f16(int math) { return math >= SXB_MATH_WMMA_F16 && math <= SXB_MATH_WMMA_F16_WIDE256; }
inline bool math_ok(int math) { return math >= SXB_MATH_F32 && math <= SXB_MATH_WMMA_F16_WIDE256; }

}  // namespace sxb
