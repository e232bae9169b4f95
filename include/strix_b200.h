/* strix_b200.h - C ABI of the B200 (sm_100a) implementation of strixite's quantized MoE FFN path.
 *
 * Every entry point is the `extern "C"` twin of one launcher in the reference's namespace
 * strix::kernels (the reference file:line is cited at each declaration).  Arguments keep the
 * reference's order and meaning; what changes is only what a C ABI forces:
 *   - `const Q4DeviceView &` / `const Q8DeviceView &` become `const SxbQView *` (same fields, same order:
 *     runtime/q4_device.hpp:14-19, runtime/q8_device.hpp:13-18);
 *   - `Act`, `MoeMath` become int (SXB_ACT_*, SXB_MATH_*; kernels/norm.hpp:20, kernels/moe_grouped.hpp:39);
 *   - `hipStream_t` becomes `sxb_stream_t`, a `cudaStream_t` passed as void *;
 *   - a thrown strix::Error becomes a non-zero return code; sxb_last_error() returns the message
 *     ("function (file:line): check `cond` failed: what was expected, what was found", common/check.hpp:59-62).
 *
 * Ownership, as in the reference (kernels/moe_grouped.hpp:84-87, runtime/qwen4exp.cpp:1092-1101): the caller owns
 * every buffer - weights, activations, ids / coef, the grouping workspace, the combine's `partial`, the error
 * words.  Unless a declaration says otherwise, no entry point allocates, frees or synchronizes; all work is enqueued
 * on the caller's stream.  Exceptions: sxb_check_*_error (a blocking 12-byte copy, as the reference's).
 *
 * Error words (`err`): >= 3 zeroed uint32 on the device, zeroed by the caller at session start.  A data error on the
 * device sets err[0] = 1, err[1], err[2] (first writer wins), poisons the affected outputs with NaN and never reads
 * out of bounds (kernels/moe_router.hpp:19-23, kernels/linear_q4.hpp:39-41, kernels/moe_grouped.hpp:13-15).
 *
 * Threading: one host thread at a time per stream, as the reference's session (serve/seq_backend.hpp:7-9).  The
 * library keeps no per-device state except lazily cached function attributes, so several devices may be driven
 * from one process (one current device per call).
 */
#ifndef STRIX_B200_H
#define STRIX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with -fvisibility=hidden */
#endif

typedef void *sxb_stream_t; /* cudaStream_t */

/* Return codes. */
enum {
    SXB_OK = 0,
    SXB_ERR_CHECK = 1, /* a precondition failed before any launch (the reference throws strix::Error) */
    SXB_ERR_CUDA = 2,  /* a CUDA call or launch failed (the reference's STRIX_HIP_CHECK_LAUNCH) */
    SXB_ERR_FATAL = 3, /* a sticky CUDA error: the context is gone (the reference's GpuFatalError) */
    SXB_ERR_DATA = 4   /* sxb_check_* / sxb_report_*: the device error words are set */
};

/* kernels/norm.hpp:20  enum class Act { F32, BF16 }.  BF16 buffers hold raw uint16_t bits. */
enum {
    SXB_ACT_F32 = 0,
    SXB_ACT_BF16 = 1,
    /* Not in the reference: F16 activations laid out by sxb_stage_f16 for a tensor-core operand.  Accepted as the
     * input dtype of the WMMA_F16 grouped gathers only. */
    SXB_ACT_F16_STAGED = 2,
    /* Not in the reference: F16 activations in the tile-blocked form made by sxb_stage_f16_tiles (rows in the pack's slot
     * order, one contiguous run per 128-slot tile and k-block).  Same use as SXB_ACT_F16_STAGED, faster. */
    SXB_ACT_F16_TILED = 3
};

/* kernels/moe_grouped.hpp:39  enum class MoeMath.  Here:
 *   F32, WMMA_BF16            exact products: BF16 activations times the integer codes on mma.sync tensor cores,
 *                             scale / min applied per group in FP32, FP32 accumulation (the reference's
 *                             "exact weights" semantics; only the summation order differs from its FP32 kernels);
 *   WMMA_F16 and its kinds    activations as F16, weights dequantized to F16 (code * scale + min, one rounding),
 *                             FP32 accumulation in tensor memory on tcgen05 tensor cores, the combine's per-slot dots
 *                             stored as BF16 (kernels/moe_grouped.hip:47-57).  Narrow / Wide / Wide256 are accepted
 *                             for source compatibility and select the same kernel. */
enum {
    SXB_MATH_F32 = 0,
    SXB_MATH_WMMA_BF16 = 1,
    SXB_MATH_WMMA_F16 = 2,
    SXB_MATH_WMMA_F16_NARROW = 3,
    SXB_MATH_WMMA_F16_WIDE = 4,
    SXB_MATH_WMMA_F16_WIDE256 = 5,
    /* Not in the reference: WMMA_F16 with the combine's per-slot dots kept in FP32.  The reference's matrix-unit path
     * - and SXB_MATH_WMMA_F16 .. WIDE256 here - round them to BF16 (kernels/moe_grouped.hip:47-57). */
    SXB_MATH_WMMA_F16_F32_PARTIALS = 6
};

/* runtime/q4_device.hpp:14-19 (Q4DeviceView) and runtime/q8_device.hpp:13-18 (Q8DeviceView): a non-owning view of
 * a row-major quantized matrix W [N, K] with groups of G codes along K (formats/q4.hpp:3-8, formats/q8.hpp:3-11):
 *   Q4: q [N, K/2] bytes, low nibble = even k;   Q8: q [N, K] bytes;
 *   scale, minv [N, K/G] BF16 bits;   w[n, k] = code * scale[n, k/G] + minv[n, k/G].
 * Experts are stacked along N: expert e = rows e*N/E .. (e+1)*N/E - 1 (kernels/linear_q4.hpp:32-35). */
typedef struct SxbQView {
    const uint8_t *q;
    const uint16_t *scale;
    const uint16_t *minv;
    int64_t N, K, G;
} SxbQView;

/* kernels/moe_grouped.hpp:75-81  struct MoeSharedAdd. */
typedef struct SxbMoeSharedAdd {
    const void *s;           /* the shared expert's output [M, N] in y's dtype (the reference's y is in the activation
                                dtype; with out_act = SXB_ACT_F32 s is FP32 too), not overlapping y */
    const float *gate_logit; /* token m's gate logit at gate_logit[m * gate_ld] */
    int64_t gate_ld;
    uint32_t gate_index;
    uint32_t *err;
} SxbMoeSharedAdd;

/* The message of the calling thread's last failed call ("" if none).  Valid until that thread's next failure. */
const char *sxb_last_error(void);
/* "strix_b200 <version> sm_100a" */
const char *sxb_version(void);

/* ---- Router ------------------------------------------------------------------------------------------------ */

/* kernels/moe_router.hpp:38-40  moe_router.  Top-k on the logits (larger first, a tie to the lower index), coef =
 * softmax over the k picks; optional shared slot k (id = shared_id, coef = sigmoid(gate logit)).  ids [M, A] int32,
 * coef [M, A] F32, A = k + (shared_logit != NULL).  1 <= E <= 1024, 1 <= k <= min(E, 32), ld >= E.  A non-finite
 * logit: that token's ids -1, coef NaN, err = {1, token, expert index (E = the shared logit)}. */
int sxb_moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                   int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, int act, uint32_t *err,
                   sxb_stream_t stream);
/* kernels/moe_router.hpp:41-43  check_router_error (synchronizes: copies the 3 words) / report_router_error (the 3
 * words already on the host).  Return SXB_ERR_DATA with the reference's message when err[0] != 0. */
int sxb_check_router_error(const uint32_t *err, const char *what);
int sxb_report_router_error(const uint32_t e[3], const char *what);

/* kernels/moe_router.hpp:53-54  moe_shared_add:  y[m, :] += sigmoid(gate_logit[m * gate_ld]) * s[m, :]. */
int sxb_moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                       uint32_t gate_index, int act, uint32_t *err, sxb_stream_t stream);
/* kernels/moe_router.hpp:61-63  moe_shared_add_inject: the add, then x[m, st*N + n] = fma(w_in[m, st], y, x) for the
 * H = 4 residual streams of x [M, H*N]. */
int sxb_moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                              uint32_t gate_index, void *x, const float *w_in, int64_t H, int act, uint32_t *err,
                              sxb_stream_t stream);

/* ---- Router-logits projection (the step before the router) and residual add (the step after the block) --------- */

/* kernels/linear.hpp:22-27  linear_bf16w: y [M, N] = x [M, K] * W^T, W [N, K] raw BF16 bits, FP32 accumulation, one rounding;
 * BF16 x, out_act BF16 or F32 (the router logits stay FP32: runtime/qwen4exp.cpp:3149-3155).  One pass over W for all
 * tokens: the decode form.  K % 8 == 0; x and w 16-byte aligned. */
int sxb_linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, int act, int out_act,
                     sxb_stream_t stream);
/* No counterpart in the reference (whose router weight is BF16 and has no bias).  The same projection for the router:
 * logits [M, ld >= N] FP32 = x [M, K] BF16 * W^T + bias, W [N, K] FP32 (w_act = SXB_ACT_F32) or BF16 bits, bias [N] FP32
 * or NULL.  Streaming form (decode). */
int sxb_router_logits(const void *x, const void *w, int w_act, const float *bias, int64_t M, int64_t N, int64_t K, float *logits,
                      int64_t ld, sxb_stream_t stream);
/* kernels/linear_wmma.hpp:29-30  linear_bf16w_wmma: the multi-token form on the tensor cores (tcgen05 here).  The weight
 * is prepared once, at load time: sxb_router_prepare splits W [N, K] into `planes` BF16 planes [planes][Npad][K] (Npad = N
 * rounded up to 128; sxb_router_planes_bytes gives the size) - one plane for a BF16 weight; for an FP32 weight two planes
 * carry 16 bits of it, three all 24 - and the GEMM sums the exact BF16 products of x with every plane in FP32.  With
 * planes = 1, planes_in may be the BF16 weight [N, K] itself, unprepared.
 * K % 64 == 0.  A wait that ran out is reported by sxb_check_dense_status. */
size_t sxb_router_planes_bytes(int64_t N, int64_t K, int planes);
int sxb_router_prepare(const void *w, int w_act, int64_t N, int64_t K, int planes, void *planes_out, sxb_stream_t stream);
int sxb_router_logits_wmma(const void *x, const void *planes_in, int planes, const float *bias, int64_t M, int64_t N, int64_t K,
                           float *logits, int64_t ld, sxb_stream_t stream);
/* The single-stream case of kernels/hc.hpp:52-54 hc_inject (weight 1): out [n] BF16 = bf16(x + y), x BF16, y F32 or BF16
 * (y_act); out may be x itself.  n % 8 == 0. */
int sxb_residual_add(const void *x, const void *y, int y_act, void *out, int64_t n, sxb_stream_t stream);

/* kernels/hc.hpp:52-54  hc_inject: the residual injection that follows the block, in place:
 * X[t, s*d + j] += w_in[t, s] * y[t, j] for the H = 4 residual streams of X [T, H*d]; one rounding per element to the
 * activation dtype.  y must not overlap X.  (sxb_moe_shared_add_inject is this fused with the shared expert's gated add.) */
int sxb_hc_inject(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, int act, sxb_stream_t stream);

/* kernels/hc.hpp:36-42  hc_mix_down (Q4DeviceView / Q8DeviceView overloads): the first half of the hyper-connection mix that
 * produces the block's input.  X [T, H*d] (F32 or BF16, 16-byte aligned) -> h [T, r] = silu(a / H) for the first r rows of w,
 * w_in [T, H] = 2 sigmoid(a / H) for the next H rows (inject != 0; w_in must be NULL otherwise), inv [T, H] = the
 * per-stream inverse RMS.  w: [r (+ H), H*d], the hc_norm weight folded in; H == 4; d % 32 == 0; r <= 1024; T <= 65535.
 * All arithmetic FP32. */
int sxb_hc_mix_down_q4(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                       float *w_in, float *inv, int act, sxb_stream_t stream);
int sxb_hc_mix_down_q8(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                       float *w_in, float *inv, int act, sxb_stream_t stream);
/* kernels/hc.hpp:44-50  hc_mix_up (Q4ChunkMajorView / Q8ChunkMajorView overloads):
 * u[t, j] = (1/H) sum_s sigmoid(W_up[s*d + j] . h[t]) * X[t, s*d + j] * inv[t, s] * (1 + norm_w[s*d + j]), rounded once to the
 * activation dtype.  w_up: [H*d, r] in the CHUNK-MAJOR layout (formats/q4.hpp:41-55: 32-code chunk c of row n at
 * q[(c * N + n) * 16 or 32 bytes], group g's scale / min at [g * N + n]); r % 32 == 0, r <= 1024.  u must not overlap x. */
int sxb_hc_mix_up_q4(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                     int64_t d, void *u, int act, sxb_stream_t stream);
int sxb_hc_mix_up_q8(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                     int64_t d, void *u, int act, sxb_stream_t stream);
/* kernels/hc_wmma.hpp:29-38  hc_wmma_workspace_bytes + hc_mix_down_wmma (Q4DeviceView / Q8DeviceView overloads): hc_mix_down for
 * multi-token forwards on the tensor cores - x rounded once to F16, weights f16(code * scale + min), FP32 accumulation over
 * each stream's d inputs; inv, the stream sum, silu and sigmoid in FP32.  Same arguments as sxb_hc_mix_down_q*, plus the
 * workspace (device, 256-byte aligned) and inv_ready (inv already holds X's inverse RMS, as sxb_hc_inject_inv leaves it).
 * Here the H streams run as H experts of the tcgen05 grouped kernel, so the workspace holds more than the reference's FP32
 * partials (kernels/hc_wmma.hip:296-331): the grouping workspace (first, so sxb_check_grouped_status(ws, ..) reports a
 * device-side wait that ran out), the restacked weight, X as tile-blocked F16 and the per-slot dots.  R = r (+ H).
 * d % 128 == 0, d % G == 0, T <= 65535.  Returns 0 and sets the error message on bad arguments. */
size_t sxb_hc_mix_down_wmma_workspace_bytes(int64_t T, int64_t H, int64_t d, int64_t R, int bits, int64_t G);
int sxb_hc_mix_down_wmma_q4(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                            float *w_in, float *inv, void *ws, size_t ws_bytes, int act, int inv_ready, sxb_stream_t stream);
int sxb_hc_mix_down_wmma_q8(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                            float *w_in, float *inv, void *ws, size_t ws_bytes, int act, int inv_ready, sxb_stream_t stream);
/* kernels/hc_wmma.hpp:40-43  hc_inject_inv: sxb_hc_inject fused with the next mix's inverse RMS of the updated X into
 * inv [T, H] - the stored (rounded) values are the ones squared - in one pass over X.  H == 4. */
int sxb_hc_inject_inv(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, float eps, float *inv, int act,
                      sxb_stream_t stream);
/* kernels/hc_wmma.hpp:45-49  hc_mix_up_wmma (Q4ChunkMajorView / Q8ChunkMajorView overloads): hc_mix_up on the tensor cores -
 * h rounded once to F16, weights f16(code * scale + min), FP32 accumulation; sigmoid and the stream combine in FP32.
 * Same arguments as sxb_hc_mix_up_q*, plus a workspace (the reference's launcher needs none; this one un-chunks W_up to
 * row-major and keeps the FP32 logits z of one block of 1024 tokens there): sxb_hc_mix_up_wmma_workspace_bytes, device,
 * 256-byte aligned.  h, x, norm_w, u 16-byte aligned; d % 128 == 0.  A device-side wait that ran out is reported by
 * sxb_check_dense_status. */
size_t sxb_hc_mix_up_wmma_workspace_bytes(int64_t T, int64_t H, int64_t d, int64_t r, int bits, int64_t G);
int sxb_hc_mix_up_wmma_q4(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                          int64_t d, void *u, void *ws, size_t ws_bytes, int act, sxb_stream_t stream);
int sxb_hc_mix_up_wmma_q8(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                          int64_t d, void *u, void *ws, size_t ws_bytes, int act, sxb_stream_t stream);
/* formats/q4.hpp:55 / formats/q8.hpp:46  to_chunk_major, for a weight already on the device: the codes, scales and mins of the
 * row-major view w re-laid out chunk-major into q / scale / minv (same sizes as the source arrays; K % 32 == 0). */
int sxb_to_chunk_major(const SxbQView *w, int bits, uint8_t *q, uint16_t *scale, uint16_t *minv, sxb_stream_t stream);

/* ---- Pack (grouping of slots by expert) --------------------------------------------------------------------- */

/* kernels/moe_grouped.hpp:48  moe_route_workspace_bytes.  Returns 0 and sets the error message on bad arguments.
 * The workspace layout is this library's own (see sxb_route_layout). */
size_t sxb_moe_route_workspace_bytes(int64_t M, int64_t A, int64_t E);
/* kernels/moe_grouped.hpp:53-54  moe_group_routes: counting sort of the S = M*A slots of ids [M, A] by expert into
 * ws.  Bucket E collects ids outside [0, E) and raises err = {1, id, slot} for the first such slot in slot order.
 * Unlike the reference (whose order inside a bucket is left to its atomics), slots inside a bucket are in ascending
 * slot order, so the whole workspace is reproducible.  1 <= A <= 64, 1 <= E <= 1023, M*A <= 2^20. */
int sxb_moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, void *ws, size_t ws_bytes, uint32_t *err,
                         sxb_stream_t stream);
/* No counterpart in the reference (two launches there).  sxb_moe_router (FP32 logits, no shared slot) and
 * sxb_moe_group_routes[_ep] as ONE launch of one CTA, for batches of at most 2048 slots (M * k): the decode step's
 * routing.  E_local == E_total: all experts are here (e_lo = 0); otherwise the expert-parallel pack.  Same words out as
 * the two calls. */
int sxb_moe_route_small(const float *logits, int64_t ld, int64_t M, int64_t E_total, int64_t k, int64_t e_lo, int64_t E_local,
                        int32_t *ids, float *coef, void *ws, size_t ws_bytes, uint32_t *router_err, uint32_t *expert_err,
                        sxb_stream_t stream);
/* No counterpart in the reference.  The tcgen05 grouped kernels bound every device-side wait; one that runs out writes
 * {2, work item, role} into words 5..7 of the workspace header (zeroed by every pack) and the kernel returns.  This
 * reads the header back (it synchronizes, like sxb_check_expert_error) and returns SXB_ERR_DATA if that happened. */
int sxb_check_grouped_status(const void *ws, const char *what);
/* No counterpart in the reference (which has one GPU).  The expert-parallel form: this rank owns experts
 * [e_lo, e_lo + E_local) of E_total; bucket b = expert e_lo + b; slots of other ranks' experts and invalid ids go to
 * bucket E_local.  err is raised only for ids outside [0, E_total). */
int sxb_moe_group_routes_ep(const int32_t *ids, int64_t M, int64_t A, int64_t E_total, int64_t e_lo, int64_t E_local,
                            void *ws, size_t ws_bytes, uint32_t *err, sxb_stream_t stream);
/* Word offsets (int32 units) of the parts of a workspace for (M, A, E), for hosts that read it back:
 * out[0] = header (8 words: n_tiles8, S, E, n_tiles128, ...), out[1] = offsets [E + 2], out[2] = slots [S],
 * out[3] = tile8_bucket, out[4] = tile8_start, out[5] = tile128_bucket, out[6] = tile128_start, out[7] = total words. */
int sxb_route_layout(int64_t M, int64_t A, int64_t E, int64_t out[8]);

/* No counterpart in the reference.  Bound of every device-side wait of the tcgen05 kernels for the launches that follow
 * (process-wide; default 2 s, minimum 1 us).  A wait that runs out ends its kernel with the status words set. */
int sxb_set_wait_limit(uint64_t nanoseconds);
/* Test hook, no counterpart in the reference: slot >= 0 makes CTA 0 of the following tcgen05 launches leave that fill of
 * its weight-code ring out, so a bounded wait runs out and the kernel's give-up path runs; -1 (the default) = off. */
int sxb_test_skip_ring_slot(int slot);

/* ---- Dense quantized linear --------------------------------------------------------------------------------- */

/* kernels/linear_q4.hpp:26,30  linear_q4:  y [M, N] = x [M, K] * dequant(W)^T.  out_act == act, or BF16 x -> F32 y. */
int sxb_linear_q4(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream);
/* kernels/linear_q8.hpp:13-14  linear_q8. */
int sxb_linear_q8(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream);

/* kernels/linear_wmma.hpp:23,26  linear_q4_wmma / linear_q8_wmma: the multi-token dense projection on the tensor cores,
 * here the tcgen05 grouped kernel run as one group with the result written by its epilogue (no pack, no scratch).
 * Numerics of this library's WMMA_F16 path: x as F16, weights f16(code * scale + min), FP32 accumulation, one rounding.
 * act SXB_ACT_BF16, or SXB_ACT_F16_TILED for x staged by sxb_stage_f16_tiles with a null workspace; out_act BF16 or F32.
 * K % 128 == 0, N % 16 == 0. */
int sxb_linear_q4_wmma(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream);
int sxb_linear_q8_wmma(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream);
/* No counterpart in the reference (which runs linear_q8_wmma, then swiglu): w = [gate | up] rows, h [M, N/2] =
 * silu(g) * u from the FP32 accumulators, rounded once; h_f16 as for the grouped SwiGLU gather (3 / 4: tile-blocked for a
 * Q4 / Q8 down projection, then pass act = SXB_ACT_F16_TILED to sxb_linear_q*_wmma). */
int sxb_linear_q4_wmma_swiglu(const void *x, const SxbQView *w, void *h, int64_t M, int act, int h_f16, sxb_stream_t stream);
int sxb_linear_q8_wmma_swiglu(const void *x, const SxbQView *w, void *h, int64_t M, int act, int h_f16, sxb_stream_t stream);
/* No counterpart in the reference.  The dense tcgen05 projections have no workspace to record a wait that ran out in;
 * the record lives inside the library, one per device.  Reads it back (synchronizes), clears it, SXB_ERR_DATA if set. */
int sxb_check_dense_status(const char *what);

/* kernels/swiglu.hpp:21  swiglu: gu [rows, 2I] = [gate | up] -> h [rows, I]; BF16: h = bf16(bf16(silu(g)) * u). */
int sxb_swiglu(const void *gu, void *h, int64_t rows, int64_t I, int act, sxb_stream_t stream);

/* ---- Experts, per-slot form (decode) ------------------------------------------------------------------------ */

/* kernels/linear_q4.hpp:42-43  linear_q4_experts_gather:  y[m, a, :] = x[m, :] * W[ids[m, a]]^T. */
int sxb_linear_q4_experts_gather(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M, int64_t A,
                                 void *y, int act, uint32_t *err, sxb_stream_t stream);
/* kernels/linear_q4.hpp:55-56  linear_q4_experts_gather_swiglu:  h [M, A, N/2] = silu(gate) * up of the merged
 * [gate | up] expert rows, g and u rounded as stored, then h = stored(stored(silu(g)) * u). */
int sxb_linear_q4_experts_gather_swiglu(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M,
                                        int64_t A, void *h, int act, uint32_t *err, sxb_stream_t stream);
/* kernels/linear_q4.hpp:44-46  linear_q4_experts_combine:  y[m, :] = sum_a coef[m, a] * h[m, a, :] * W[ids[m, a]]^T.
 * out_act (not in the reference, which stores y in `act`): SXB_ACT_F32 keeps the FP32 sum unrounded. */
int sxb_linear_q4_experts_combine(const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef,
                                  int64_t M, int64_t A, void *y, int act, int out_act, uint32_t *err,
                                  sxb_stream_t stream);
/* The same three for Q8 experts.  No counterpart in the reference (its experts are Q4 / Q5 only:
 * runtime/qweight.hpp:80-100); same semantics with codes 0..255. */
int sxb_linear_q8_experts_gather(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M, int64_t A,
                                 void *y, int act, uint32_t *err, sxb_stream_t stream);
int sxb_linear_q8_experts_gather_swiglu(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M,
                                        int64_t A, void *h, int act, uint32_t *err, sxb_stream_t stream);
int sxb_linear_q8_experts_combine(const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef,
                                  int64_t M, int64_t A, void *y, int act, int out_act, uint32_t *err,
                                  sxb_stream_t stream);
/* kernels/linear_q4.hpp:59-61  check_expert_error / report_expert_error. */
int sxb_check_expert_error(const uint32_t *err, const char *what);
int sxb_report_expert_error(const uint32_t e[3], const char *what);

/* ---- Experts, grouped form (multi-token forwards) ----------------------------------------------------------- */

/* kernels/moe_grouped.hpp:58-60  linear_q4_experts_gather_grouped (ws from sxb_moe_group_routes, same ids/M/A/E). */
int sxb_linear_q4_experts_gather_grouped(const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                                         int64_t M, int64_t A, void *y, int act, int math, sxb_stream_t stream);
/* kernels/moe_grouped.hpp:67-69  linear_q4_experts_gather_grouped_swiglu.  With a WMMA_F16 math: h = silu(g) * u from
 * the FP32 accumulators, rounded once.  h_f16 (WMMA_F16 only): 0 = h stored as BF16; 1 = h stored as F16 bits of its
 * BF16 rounding (the reference's h_f16); 2 = the same values with every 8 consecutive columns in the order
 * [0 4 1 5 2 6 3 7], the k order of a Q4 tensor-core operand, so the Q4 down GEMM can copy h rows without touching
 * them (pass the same h_f16 to the combine); 3 / 4 = tile-blocked for a Q4 / Q8 down operand (sxb_stage_f16_tiles).  With SXB_MATH_F32 / WMMA_BF16 (an extension: the reference refuses them
 * here) the decode form's rounding points are kept.  act may be SXB_ACT_F16_STAGED: x then holds the F16 copy made by
 * sxb_stage_f16 for this weight's bit width. */
int sxb_linear_q4_experts_gather_grouped_swiglu(const void *x, const SxbQView *w, int64_t E, const void *ws,
                                                size_t ws_bytes, int64_t M, int64_t A, void *h, int act, int math,
                                                sxb_stream_t stream, int h_f16);
/* kernels/moe_grouped.hpp:88-91  linear_q4_experts_combine_grouped.  partial: M*A*N FP32 scratch owned by the caller
 * (the per-slot dots; with a WMMA_F16 math they are stored as BF16 in the first half of it, as the reference does);
 * y[m, :] = sum_a fma(coef[m, a], partial[m*A + a, :]) in slot order, one rounding, optionally + sigmoid(gate) * s
 * (shared).  out_act as for sxb_linear_q4_experts_combine. */
int sxb_linear_q4_experts_combine_grouped(const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                                          const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                          int64_t M, int64_t A, void *y, int act, int out_act, int math,
                                          sxb_stream_t stream, const SxbMoeSharedAdd *shared, int h_f16);
/* No counterpart in the reference.  sxb_linear_q4_experts_combine_grouped for callers that cannot supply `partial`: an
 * engine whose memory plan left no spare device memory, or a decode loop that must not call cudaMalloc (it synchronizes
 * the device).  The per-slot dots go to a 16 MiB array inside the library image instead; x / h / y stay the caller's.
 * Refuses M * A * N > 4 Mi floats (4,194,304) with SXB_ERR_CHECK.  Calls no allocator.  The 16 MiB are taken when the CUDA
 * runtime loads this part of the library on a device - with its default lazy loading, inside the FIRST call on that
 * device, which also looks the array's address up (a blocking runtime call): make one small call per device before the
 * host sizes its memory plan and before any stream capture.  The address is kept per device for the life of the process (a
 * cudaDeviceReset invalidates it).  Every call on a device shares the array: calls that overlap on the GPU race. */
int sxb_linear_q4_experts_combine_grouped_noalloc(const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                                                  const float *coef, const void *ws, size_t ws_bytes, int64_t M, int64_t A,
                                                  void *y, int act, int out_act, int math, sxb_stream_t stream,
                                                  const SxbMoeSharedAdd *shared, int h_f16);
/* The same three for Q8 experts (no counterpart in the reference, see above). */
int sxb_linear_q8_experts_gather_grouped(const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                                         int64_t M, int64_t A, void *y, int act, int math, sxb_stream_t stream);
int sxb_linear_q8_experts_gather_grouped_swiglu(const void *x, const SxbQView *w, int64_t E, const void *ws,
                                                size_t ws_bytes, int64_t M, int64_t A, void *h, int act, int math,
                                                sxb_stream_t stream, int h_f16);
int sxb_linear_q8_experts_combine_grouped(const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                                          const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                          int64_t M, int64_t A, void *y, int act, int out_act, int math,
                                          sxb_stream_t stream, const SxbMoeSharedAdd *shared, int h_f16);

/* No counterpart in the reference (one GPU).  The combine for an expert-parallel rank that holds experts
 * [e_lo, e_lo + E_local) of E_total in w (ws from sxb_moe_group_routes_ep): slots routed to other ranks' experts add
 * nothing, so y is this rank's partial sum of every token's row (zeros for tokens it serves no expert of); an id
 * outside [0, E_total) still makes the row NaN. */
int sxb_linear_q4_experts_combine_grouped_ep(const void *h, const SxbQView *w, int64_t E_local, int64_t E_total,
                                             int64_t e_lo, const int32_t *ids, const float *coef, const void *ws,
                                             size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act,
                                             int out_act, int math, sxb_stream_t stream, int h_f16);
int sxb_linear_q8_experts_combine_grouped_ep(const void *h, const SxbQView *w, int64_t E_local, int64_t E_total,
                                             int64_t e_lo, const int32_t *ids, const float *coef, const void *ws,
                                             size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act,
                                             int out_act, int math, sxb_stream_t stream, int h_f16);

/* No counterpart in the reference (its kernels convert BF16 -> F16 while staging every tile, kernels/moe_grouped.hip:29-32).
 * x [M, K] BF16 -> xh [M, K] F16, every 8 consecutive k in the order a `bits`-bit weight operand uses on the tensor
 * cores ([0 4 1 5 2 6 3 7] for Q4, natural for Q8).  Done once per layer, it lets the grouped GEMMs copy activation rows
 * asynchronously instead of converting them per tile.  xh: caller-owned, M*K*2 bytes, 16-byte aligned. */
int sxb_stage_f16(const void *x, int64_t M, int64_t K, int bits, void *xh, sxb_stream_t stream);
/* No counterpart in the reference.  The tile-blocked form of the same: for a grouping workspace ws (after the pack), xs
 * receives, for every slot position pos of the slot order and every k-block kb of 64, the 128-byte F16 line of token
 * slots[pos] / A at byte (kb * S + pos) * 128, swizzled for its place in its 128-slot tile, so that a tile's operand of a
 * k-block is one contiguous run and reaches shared memory with a single bulk copy.  xs: caller-owned, M*A*K*2 bytes.
 * ws == NULL (with A = E = 1): the rows of a dense projection in their own order, for sxb_linear_q*_wmma[_swiglu].
 * Pass act = SXB_ACT_F16_TILED to the grouped gather.  The SwiGLU gather writes h in the same form with h_f16 = 3 (Q4
 * down) or 4 (Q8 down); pass the same h_f16 to the combine. */
int sxb_stage_f16_tiles(const void *x, const void *ws, size_t ws_bytes, int64_t M, int64_t A, int64_t E, int64_t K, int bits,
                        void *xs, sxb_stream_t stream);

/* ---- The whole block as one call ---------------------------------------------------------------------------- */

/* One MoE block: what runtime/qwen4exp.cpp:3143-3217 issues launcher by launcher - router top-k, grouping, gate/up +
 * SwiGLU, down + combine, the shared expert folded into the combine - as one entry point on one stream.  Every buffer is
 * the caller's (sizes below; the reference's session buffers, runtime/qwen4exp.cpp:1018-1027,1092-1101); nothing is
 * allocated and nothing synchronizes.  The rounding points are those of the entry points it calls. */
typedef struct SxbMoeLayerArgs {
    int64_t M;                     /* tokens */
    int64_t E, A;                  /* experts in the weight views; active experts per token */
    int64_t E_total, e_lo;         /* E_total == E: all experts are here.  Otherwise the views hold experts [e_lo, e_lo + E) of
                                      E_total (an expert-parallel rank) and y receives this rank's partial sums */
    const SxbQView *gate_up, *down;/* stacked experts [E * 2I, d] and [E * d, I] */
    int gate_up_bits, down_bits;   /* 4 or 8 */
    const SxbQView *shared_gate_up, *shared_down; /* the always-on shared expert [2I, d], [d, I]; NULL, NULL = none */
    int shared_bits;
    const void *x;                 /* [M, d] BF16 */
    const float *logits;           /* [M, logits_ld] FP32 router logits; with a shared expert column E_total is its gate.
                                      NULL: ids and coef already hold the routes and no router runs */
    int64_t logits_ld;
    void *y;                       /* [M, d] */
    int out_act;                   /* SXB_ACT_BF16, or SXB_ACT_F32 for the unrounded sums */
    int math;                      /* SXB_MATH_*; -1 = the tcgen05 kernels (FP32 per-slot dots) from 256 tokens up, the streaming ones below */
    /* work buffers */
    int32_t *ids;                  /* [M, A] */
    float *coef;                   /* [M, A] */
    void *ws;                      /* sxb_moe_route_workspace_bytes(M, A, E) */
    size_t ws_bytes;
    void *h;                       /* [M * A, I] 16-bit */
    float *partial;                /* [M * A, d] */
    void *xs;                      /* [M * A, d] F16: tile-blocked activations; tcgen05 path only (else may be NULL) */
    void *sh_gu, *sh_h;            /* shared expert: [M, 2I] (streaming path only), [M, I], 16-bit */
    void *sh_y;                    /* shared expert's output [M, d] in y's dtype */
    int32_t *sh_ids;               /* unused (kept for layout compatibility): the shared expert's prefill form is a dense */
    float *sh_coef;                /* tcgen05 projection and needs no routes, workspace or scratch; may be NULL */
    void *sh_ws;
    size_t sh_ws_bytes;
    float *sh_partial;
    void *sh_xs;                   /* [M, d] F16: tcgen05 path with a shared expert only */
    uint32_t *router_err, *expert_err; /* >= 3 words each, zeroed by the caller at session start */
} SxbMoeLayerArgs;
int sxb_moe_layer(const SxbMoeLayerArgs *args, sxb_stream_t stream);

/* ---- Expert parallelism (no counterpart in the reference, which drives one GPU) ------------------------------- */

/* One process per GPU; rank r of `world` holds experts [r E / world, (r + 1) E / world) of every layer and owns the token
 * rows [r T / world, (r + 1) T / world).  sxb_moe_layer_ep runs one layer on the rank's rows: all-gather of the activations
 * and of the routes (NCCL), this rank's experts on all T rows, and the rows' way back to their owners:
 *   return_path 0  the partial rows [T, d] FP32 through ncclReduceScatter (sum);
 *   return_path 1  every row stored, as the rank's piece, straight into its owner's receive buffer through peer-mapped
 *                  pointers (plain stores from the combine kernel), the owner adds its `world` pieces in rank order (FP32);
 *   return_path 2  the same with F16 pieces (half the bytes on the links; one rounding to 11 bits per piece; |piece| < 65504).
 * libnccl.so.2 is opened at run time, not linked.  sxb_ep_unique_id: rank 0 makes the communicator's id and the host sends
 * the 128 bytes to the other ranks by its own means.  sxb_ep_create (collective, synchronizes) builds the communicator,
 * allocates the rank's exchange buffers ONCE (device memory: T*d*2 bytes of gathered activations, plus T*d*4 (paths 0, 1) or
 * T*d*2 (path 2)) and maps the peers' receive buffers (CUDA IPC).  The per-layer call allocates nothing and uses the
 * caller's stream plus one stream of the library's for the activation gather. */
typedef struct SxbEp SxbEp;
int sxb_ep_unique_id(uint8_t id[128]);
int sxb_ep_create(const uint8_t id[128], int world, int rank, int64_t T, int64_t d, int64_t A, int return_path, SxbEp **out);
int sxb_ep_destroy(SxbEp *ep);
/* args as for sxb_moe_layer with: M = the rank's rows t = T / world; x [t, d], logits [t, ld] and y [t, d] the rank's rows
 * (y = the full sums over every rank's experts, FP32 or BF16); E, e_lo, E_total the rank's experts; no shared expert (it is
 * not sharded: run it on the rows' owner).  The work buffers ids, coef, ws, h, partial, xs are sized for all T rows. */
int sxb_moe_layer_ep(SxbEp *ep, const SxbMoeLayerArgs *args, sxb_stream_t stream);
/* Phase timing for tuning: on = 1 records CUDA events at the phase boundaries of the following calls; sxb_ep_timing
 * (synchronizes) returns the mean milliseconds a layer of {routing + route gather, wait for the activations, experts issued,
 * exchange back, sum of the pieces} over the last `*layers` (at most 64) calls. */
int sxb_ep_set_timing(SxbEp *ep, int on);
int sxb_ep_timing(SxbEp *ep, float ms[5], int *layers);

/* ---- strixw: the converted-weights file (formats/strixw.hpp:17-50) ---------------------------------------------- */

/* formats/strixw.hpp:13-16  StrixwEncoding / StrixwRole. */
enum { SXB_STRIXW_Q4 = 1, SXB_STRIXW_Q4_CHUNK_MAJOR = 2, SXB_STRIXW_BF16 = 3, SXB_STRIXW_F32 = 4, SXB_STRIXW_I64 = 5,
       SXB_STRIXW_Q8 = 6, SXB_STRIXW_Q8_CHUNK_MAJOR = 7, SXB_STRIXW_Q6 = 8, SXB_STRIXW_Q5 = 9 };
enum { SXB_STRIXW_DATA = 0, SXB_STRIXW_QCODES = 1, SXB_STRIXW_SCALE = 2, SXB_STRIXW_MIN = 3 };
/* formats/strixw.hpp:37-48  StrixwTensor, flattened (name points into the file object; parts through sxb_strixw_part). */
typedef struct SxbStrixwTensor {
    const char *name;
    int encoding, ndim;
    int64_t shape[8];
    int64_t group_size, experts;
    int n_parts, n_components;
    int component_role[3];
    uint64_t component_offset[3], component_bytes[3], component_hash[3]; /* offsets: absolute, in the file */
} SxbStrixwTensor;
typedef struct SxbStrixw SxbStrixw;
/* formats/strixw.hpp:96-120  StrixwFile: maps the file and validates header, index and every record (versions 1..4). */
int sxb_strixw_open(const char *path, SxbStrixw **out);
int sxb_strixw_close(SxbStrixw *f);
int64_t sxb_strixw_tensor_count(const SxbStrixw *f);
int sxb_strixw_tensor(const SxbStrixw *f, int64_t index, SxbStrixwTensor *out);
int sxb_strixw_find(const SxbStrixw *f, const char *name, SxbStrixwTensor *out);
int sxb_strixw_part(const SxbStrixw *f, const char *name, int index, const char **source, int64_t *row_offset, int64_t *rows);
const char *sxb_strixw_meta(const SxbStrixw *f, const char *key);             /* NULL if absent */
const void *sxb_strixw_data(const SxbStrixw *f, const char *name, int role);  /* host pointer into the mapping; NULL if absent */
/* StrixwFile::verify_hashes: recomputes every component hash on `threads` host threads. */
int sxb_strixw_verify(const SxbStrixw *f, int threads);
/* formats/strixw.hpp:58  strix_hash64. */
uint64_t sxb_strix_hash64(const void *data, size_t n);
/* runtime/strixw_loader.hpp:37-60  StrixwDevice: the whole data region as ONE device allocation (made here, once), filled
 * through two pinned staging buffers by `read_threads` concurrent pread()s and asynchronous copies on `stream`; returns
 * when the data is resident.  Components keep their file offsets (4096 / 256-byte alignment carries over). */
int sxb_strixw_load(SxbStrixw *f, int read_threads, sxb_stream_t stream);
double sxb_strixw_load_seconds(const SxbStrixw *f);
const void *sxb_strixw_device_ptr(const SxbStrixw *f, const char *name, int role);
/* StrixwDevice::q4 / q8 / qw: the device view of a Q4 or Q8 row-major tensor of the expected shape; *bits = 4 or 8. */
int sxb_strixw_qview(const SxbStrixw *f, const char *name, int64_t N, int64_t K, SxbQView *view, int *bits);
/* formats/merge_plan.cpp:33-41: "<layer>mlp.experts_gate_up" / "<layer>mlp.experts_down" stack the E routed experts and,
 * when it shares their format, the shared expert as expert #E.  routed = the view of the E routed experts; shared (may be
 * NULL) = the shared expert's view, or all zero when the file keeps it elsewhere. */
int sxb_strixw_expert_views(const SxbStrixw *f, const char *name, int64_t E, SxbQView *routed, SxbQView *shared, int *bits);

/* ---- Quantizers on the device ------------------------------------------------------------------------------- */

/* formats/q4.hpp:32 quantize_q4 / formats/q8.hpp:32 quantize_q8, for weights already on the device: w [N, K] FP32 ->
 * codes, scales, mins, bit-identical to the reference's host quantizers (IEEE division, round half to even).
 * bits = 4 or 8; G = 32, 64 or 128; K % G == 0.  Non-finite input sets err = {1, row, column}. */
int sxb_quantize(const float *w, int64_t N, int64_t K, int64_t G, int bits, uint8_t *q, uint16_t *scale,
                 uint16_t *minv, uint32_t *err, sxb_stream_t stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* STRIX_B200_H */
