// Act::F32 activations into the quantized projections (kernels/linear_q4.hpp:26-30, kernels/moe_grouped.hpp:29: "the
// engine's default semantics"): x, h and the outputs are FP32, the weights are the FP32 dequantization
// code * scale + min (two roundings, formats/q4.cpp:121-134), sums in FP32.  The served models run BF16 activations, so
// this is a plain correctness path - one warp per output element, lanes strided over k - not a tuned one: every
// sxb_linear_q* / sxb_linear_q*_experts_* entry point takes it when its `act` is SXB_ACT_F32.

#include "experts.cuh"

#include <algorithm>

namespace sxb {
namespace {

constexpr int kWarps = 8;

struct F32Args {
    const float *x;      // activations, row r at x + r * K
    const uint8_t *q;
    const uint16_t *scale, *minv;
    int64_t N, K, G;     // rows per expert, codes per row, group size
    int64_t rows;        // rows of work: slots, positions of the slot order, or tokens
    int64_t A, E;
    const int32_t *ids;  // per-slot ids (by_ws == 0)
    const int32_t *ws;   // grouping workspace (by_ws == 1): rows are positions of the slot order
    RouteWords L;
    const float *coef;   // combine
    float *out;
    uint32_t *err;
    int row_div;         // activation row of slot s is s / row_div (A for x rows, 1 for h rows)
    int64_t row0;        // first row of work of this launch (grid.y holds at most 65535 rows)
};

template <int BITS>
__device__ inline float weight_at(const F32Args &a, int64_t row, int64_t k) {
    const int64_t g = row * (a.K / a.G) + k / a.G;
    const float s = bf16_bits_to_f32(a.scale[g]), m = bf16_bits_to_f32(a.minv[g]);
    int code;
    if (BITS == 8) code = a.q[row * a.K + k];
    else code = (a.q[(row * a.K + k) >> 1] >> ((k & 1) ? 4 : 0)) & 0xF;
    return __fadd_rn(__fmul_rn((float)code, s), m);
}

template <int BITS>
__device__ inline float warp_dot(const F32Args &a, const float *xr, int64_t wrow, int lane) {
    float acc = 0.f;
    for (int64_t k = lane; k < a.K; k += 32) acc = fmaf(xr[k], weight_at<BITS>(a, wrow, k), acc);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    return acc;
}

// (slot, expert id) of work row r.  id outside [0, E): the slot's outputs become NaN.
__device__ inline void slot_of(const F32Args &a, int64_t r, int64_t *slot, int32_t *id) {
    if (a.ws == nullptr) {
        *slot = r;
        *id = a.ids ? a.ids[r] : 0;
        return;
    }
    // position r of the slot order: the bucket whose range of offsets holds it
    const int32_t *off = a.ws + a.L.offsets;
    int lo = 0, hi = (int)a.E + 1;  // off[lo] <= r < off[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (off[mid] <= r) lo = mid;
        else hi = mid;
    }
    *slot = a.ws[a.L.slots + r];
    *id = lo;  // bucket E holds the slots whose id was out of range
}

// MODE 0: out[slot, n] = x_row . W[id][n];  MODE 1: out[slot, j] = silu(x_row . gate_j) * (x_row . up_j)
template <int BITS, int MODE>
__global__ void __launch_bounds__(32 * kWarps) f32_gather_kernel(const F32Args a) {
    const int lane = threadIdx.x & 31;
    const int64_t cols = MODE == 1 ? a.N / 2 : a.N;
    const int64_t n = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5), r = a.row0 + blockIdx.y;
    if (n >= cols) return;
    int64_t slot;
    int32_t id;
    slot_of(a, r, &slot, &id);
    const bool ok = id >= 0 && id < a.E;
    if (!ok && a.err != nullptr && n == 0 && lane == 0) raise_error(a.err, (uint32_t)id, (uint32_t)slot);
    float v = qnan_f32();
    if (ok) {
        const float *xr = a.x + (slot / a.row_div) * a.K;
        const int64_t wrow = (int64_t)id * a.N + n;
        v = warp_dot<BITS>(a, xr, wrow, lane);
        if (MODE == 1) v = silu_f32(v) * warp_dot<BITS>(a, xr, wrow + a.N / 2, lane);
    }
    if (lane == 0) a.out[slot * cols + n] = v;
}

// out[m, n] = sum_a fma(coef[m, a], h[m*A + a] . W[ids[m, a]][n]) in slot order (kernels/linear_q4.hip:281-322)
template <int BITS>
__global__ void __launch_bounds__(32 * kWarps) f32_combine_kernel(const F32Args a) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5), m = blockIdx.y;
    if (n >= a.N) return;
    float acc = 0.f;
    bool ok = true;
    for (int64_t k = 0; k < a.A; ++k) {
        const int32_t id = a.ids[m * a.A + k];
        if (id < 0 || id >= a.E) {
            if (ok && n == 0 && lane == 0) raise_error(a.err, (uint32_t)id, (uint32_t)(m * a.A + k));
            ok = false;
            continue;
        }
        acc = fmaf(a.coef[m * a.A + k], warp_dot<BITS>(a, a.x + (m * a.A + k) * a.K, (int64_t)id * a.N + n, lane), acc);
    }
    if (lane == 0) a.out[m * a.N + n] = ok ? acc : qnan_f32();
}

int check_f32(const char *fn, const void *x, const SxbQView *w, const void *out, int64_t E) {
    SXB_CHECK(x != nullptr && out != nullptr && w != nullptr, fn, ": null pointer (x=", x, ", out=", out, ")");
    SXB_CHECK(w->q != nullptr && w->scale != nullptr && w->minv != nullptr, fn, ": null weight pointer");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->K >= w->G && w->K % w->G == 0 && w->K <= (1 << 24), fn, ": K = ", w->K, " must be a positive multiple of G = ", w->G);
    SXB_CHECK(E >= 1 && w->N % E == 0, fn, ": weight has ", w->N, " rows for E = ", E, " experts");
    return SXB_OK;
}

}  // namespace

// mode 0 plain, 1 SwiGLU.  ids == nullptr and ws == nullptr: dense (rows = M tokens, expert 0).
template <int BITS>
int f32_gather(const char *fn, const void *x, const SxbQView *w, int64_t E, const int32_t *ids, const void *ws, int64_t M, int64_t A,
               void *y, bool swiglu, int row_div, uint32_t *err, sxb_stream_t stream) {
    if (int rc = check_f32(fn, x, w, y, E)) return rc;
    const int64_t rows = M * A;
    SXB_CHECK(rows >= 1 && rows <= 0x7fffffff / 2, fn, ": ", rows, " rows of work");
    F32Args a{};
    a.x = static_cast<const float *>(x), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = w->N / E, a.K = w->K, a.G = w->G, a.rows = rows, a.A = A, a.E = E, a.ids = ids, a.ws = static_cast<const int32_t *>(ws);
    if (ws) a.L = route_words(M, A, E);
    a.out = static_cast<float *>(y), a.err = err, a.row_div = row_div;
    SXB_CHECK(!swiglu || a.N % 2 == 0, fn, ": [gate | up] rows: ", a.N, " rows an expert must be even");
    const int64_t cols = swiglu ? a.N / 2 : a.N;
    auto st = static_cast<cudaStream_t>(stream);
    for (int64_t r0 = 0; r0 < rows; r0 += 65535) {  // grid.y is limited to 65535: larger row counts go in slices
        a.row0 = r0;
        const dim3 grid((unsigned)((cols + kWarps - 1) / kWarps), (unsigned)std::min<int64_t>(65535, rows - r0));
        if (swiglu) f32_gather_kernel<BITS, 1><<<grid, 32 * kWarps, 0, st>>>(a);
        else f32_gather_kernel<BITS, 0><<<grid, 32 * kWarps, 0, st>>>(a);
    }
    SXB_CHECK_LAUNCH(fn, " F32 activations rows=", rows, " N=", a.N, " K=", a.K);
    return SXB_OK;
}

template <int BITS>
int f32_combine(const char *fn, const void *h, const SxbQView *w, int64_t E, const int32_t *ids, const float *coef, int64_t M,
                int64_t A, void *y, uint32_t *err, sxb_stream_t stream) {
    if (int rc = check_f32(fn, h, w, y, E)) return rc;
    SXB_CHECK(ids != nullptr && coef != nullptr && err != nullptr, fn, ": null pointer (ids / coef / err)");
    SXB_CHECK(M >= 1 && M <= 65535, fn, ": M (tokens) = ", M, ", expected 1..65535");
    F32Args a{};
    a.x = static_cast<const float *>(h), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = w->N / E, a.K = w->K, a.G = w->G, a.rows = M, a.A = A, a.E = E, a.ids = ids, a.coef = coef;
    a.out = static_cast<float *>(y), a.err = err, a.row_div = 1;
    const dim3 grid((unsigned)((a.N + kWarps - 1) / kWarps), (unsigned)M);
    f32_combine_kernel<BITS><<<grid, 32 * kWarps, 0, static_cast<cudaStream_t>(stream)>>>(a);
    SXB_CHECK_LAUNCH(fn, " F32 activations M=", M, " A=", A, " N=", a.N, " K=", a.K);
    return SXB_OK;
}

template int f32_gather<4>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const void *, int64_t, int64_t, void *,
                           bool, int, uint32_t *, sxb_stream_t);
template int f32_gather<8>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const void *, int64_t, int64_t, void *,
                           bool, int, uint32_t *, sxb_stream_t);
template int f32_combine<4>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const float *, int64_t, int64_t,
                            void *, uint32_t *, sxb_stream_t);
template int f32_combine<8>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const float *, int64_t, int64_t,
                            void *, uint32_t *, sxb_stream_t);

}  // namespace sxb
