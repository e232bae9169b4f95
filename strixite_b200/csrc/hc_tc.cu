// The hyper-connection mix for multi-token forwards on the tensor cores (kernels/hc_wmma.hpp:34-47, kernels/hc_wmma.hip):
// the same math and weight layouts as hc.cu's per-token forms, with the numerics of the reference's matrix-unit path -
// x and h rounded once to F16, the weights dequantized to F16 (code * scale + min, one rounding), FP32 accumulation over
// each product's whole K range; norms, gates and the stream combine in FP32.
//
// Both halves run on this library's tcgen05 expert kernels rather than on kernels of their own:
//   down  a = sum_s inv[t, s] * (W'_s . X_s[t]) is a grouped projection with the H streams as H "experts": slot t * H + s
//         holds the row X_s[t] (X [T, H*d] read as [T*H, d] IS that slot-major matrix), expert s the weight's column range
//         [s d, (s + 1) d) restacked as rows [s Rp, (s + 1) Rp) of a [H * Rp, d] view (Rp = R rounded up to 16, the padding
//         rows zero).  One pass over X computes inv and writes the tile-blocked F16 operand; the grouping workspace of that
//         regular pattern is written directly (no ids, no sort); the grouped kernel leaves FP32 per-slot dots; a last pass folds them with
//         inv, in stream order (kernels/hc_wmma.hip:136-150), into h and w_in.
//   up    z = h W_up^T is a dense projection of h [T, r] on W_up [H*d, r], un-chunked to row-major with r padded to a
//         multiple of 128 by zero groups and its rows put in the order that makes the four streams of an output column
//         neighbours in tensor memory; the kernel's epilogue is the stream combine itself,
//         u = (1/H) sum_s sigmoid(z_s) * X_s * inv_s * (1 + norm_w_s) (kernels/hc_wmma.hip:244-272), so z never exists
//         in memory.
// The re-layouts of the two weights (a few MB) are done per call into the caller's workspace: the views an engine holds
// stay the reference's (row-major folded down weight, chunk-major up weight), shared with the per-token kernels.

#include "experts.cuh"
#include "route_pack.cuh"
#include "tc_ptx.cuh"

#include <algorithm>
#include <cmath>

namespace sxb {
namespace {

constexpr int kStreams = 4;
constexpr int kChunk = 32;           // codes per chunk of the chunk-major layout
constexpr int64_t kMaxRank = 1024;

inline int64_t up16(int64_t v) { return (v + 15) / 16 * 16; }
inline int64_t up128(int64_t v) { return (v + 127) / 128 * 128; }
inline size_t al256(size_t v) { return (v + 255) / 256 * 256; }

// Eight FP32 values -> one 16-byte chunk of F16 in the k order of a BITS-bit weight operand ([0 4 1 5 2 6 3 7] for Q4).
template <int BITS>
__device__ inline uint4 f16_chunk(const float (&f)[8]) {
    uint4 o;
    if (BITS == 4) {
        o.x = h2_as_u32(__floats2half2_rn(f[0], f[4])), o.y = h2_as_u32(__floats2half2_rn(f[1], f[5]));
        o.z = h2_as_u32(__floats2half2_rn(f[2], f[6])), o.w = h2_as_u32(__floats2half2_rn(f[3], f[7]));
    } else {
        o.x = h2_as_u32(__floats2half2_rn(f[0], f[1])), o.y = h2_as_u32(__floats2half2_rn(f[2], f[3]));
        o.z = h2_as_u32(__floats2half2_rn(f[4], f[5])), o.w = h2_as_u32(__floats2half2_rn(f[6], f[7]));
    }
    return o;
}
// Eight consecutive activations starting at element i (a multiple of 8) as FP32.
__device__ inline void load8(const float *p, int64_t i, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p + i)), b = __ldg(reinterpret_cast<const float4 *>(p + i) + 1);
    f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}
__device__ inline void load8(const uint16_t *p, int64_t i, float (&f)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4 *>(p + i));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) f[2 * j] = __uint_as_float(w[j] << 16), f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
}

// ---- down ----------------------------------------------------------------------------------------------------------

// The folded down weight [R, H*d] -> per-stream stacks [H * Rp, d]: codes, scales and mins of columns [s d, (s + 1) d) of
// row n become row s * Rp + n; rows n >= R are zero codes with zero scale and min.
__global__ void __launch_bounds__(256) hc_stack_down_kernel(const uint8_t *__restrict__ q, const uint16_t *__restrict__ scale,
                                                            const uint16_t *__restrict__ minv, int64_t R, int64_t Rp, int64_t d, int64_t G,
                                                            int bits, uint32_t *__restrict__ qo, uint16_t *__restrict__ so,
                                                            uint16_t *__restrict__ mo) {
    const int64_t row_vecs = d * bits / 128, row_groups = d / G, stride = (int64_t)gridDim.x * blockDim.x;  // 16-byte pieces a stream's row
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint4 *qi = reinterpret_cast<const uint4 *>(q);
    uint4 *qv = reinterpret_cast<uint4 *>(qo);
    for (int64_t i = first; i < kStreams * Rp * row_vecs; i += stride) {
        const int64_t w = i % row_vecs, sn = i / row_vecs, n = sn % Rp, s = sn / Rp;
        qv[i] = n < R ? __ldg(qi + (n * kStreams + s) * row_vecs + w) : make_uint4(0u, 0u, 0u, 0u);
    }
    for (int64_t i = first; i < kStreams * Rp * row_groups; i += stride) {
        const int64_t g = i % row_groups, sn = i / row_groups, n = sn % Rp, s = sn / Rp;
        const int64_t at = (n * kStreams + s) * row_groups + g;
        so[i] = n < R ? scale[at] : (uint16_t)0, mo[i] = n < R ? minv[at] : (uint16_t)0;
    }
}

// One pass over X [T, H*d]: inv[t, s] = 1 / sqrt(mean(X_s[t]^2) + eps) (kernels/hc_wmma.hip:25-45; skipped when the caller
// has it), and the row X_s[t] as F16 in the tile-blocked form at the position the pack gives slot t * H + s: bucket s
// starts at s * T and holds its slots in ascending order, and a row's swizzle depends on its place in its tile modulo 8
// only, which is t modulo 8 for every tile size in use.  A warp per row, rows in position order.
template <typename TX, int BITS>
__global__ void __launch_bounds__(256) hc_stage_down_kernel(const TX *__restrict__ x, int64_t T, int64_t d, float eps, bool want_inv,
                                                            float *__restrict__ inv, unsigned char *__restrict__ xs) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5), S = T * kStreams;
    const int chunks = (int)(d / 8);
    for (int64_t pos = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); pos < S; pos += warps) {
        const int64_t s = pos / T, t = pos % T;
        const TX *row = x + (t * kStreams + s) * d;
        float ssq = 0.f;
        for (int k8 = lane; k8 < chunks; k8 += 128) {
            float f[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (k8 + 32 * u < chunks) load8(row, (int64_t)(k8 + 32 * u) * 8, f[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kk = k8 + 32 * u;
                if (kk < chunks) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) ssq = fmaf(f[u][j], f[u][j], ssq);
                    *reinterpret_cast<uint4 *>(xs + tiled_offset(S, kk >> 3, pos, (int)(t & 7), kk & 7)) = f16_chunk<BITS>(f[u]);
                }
            }
        }
        if (want_inv) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) inv[t * kStreams + s] = 1.0f / sqrtf(ssq / (float)d + eps);
        }
    }
}

// a = sum_s inv[t, s] * P[t * H + s, n] in stream order, z = a / H, h = silu(z) for n < r, w_in = 2 sigmoid(z) after
// (kernels/hc_wmma.hip:136-150).
__global__ void __launch_bounds__(256) hc_finish_down_kernel(const float *__restrict__ partial, const float *__restrict__ inv, int64_t T,
                                                             int64_t R, int64_t Rp, int64_t r, float *__restrict__ h,
                                                             float *__restrict__ w_in) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * R) return;
    const int64_t t = i / R, n = i % R;
    float a = 0.f;
#pragma unroll
    for (int s = 0; s < kStreams; ++s) a = fmaf(inv[t * kStreams + s], partial[(t * kStreams + s) * Rp + n], a);
    const float z = a / (float)kStreams;
    if (n < r) h[t * r + n] = z / (1.0f + expf(-z));
    else w_in[t * kStreams + (n - r)] = 2.0f / (1.0f + expf(-z));
}

// ---- inject + inv --------------------------------------------------------------------------------------------------

// kernels/hc_wmma.hip:47-73 hc_inject_inv: X[t, s d + j] = stored(fma(w_in[t, s], y[t, j], X[t, s d + j])) and inv[t, s]
// from the stored values, in one pass.  A CTA per token; a thread takes columns j and updates their four streams.
template <typename TX>
__global__ void __launch_bounds__(256) hc_inject_inv_kernel(TX *__restrict__ x, const float *__restrict__ w_in, const TX *__restrict__ y,
                                                            int64_t d, float eps, float *__restrict__ inv) {
    __shared__ float red[kStreams][8];
    const int64_t t = blockIdx.x;
    TX *xr = x + t * kStreams * d;
    float wi[kStreams], ssq[kStreams] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < kStreams; ++s) wi[s] = w_in[t * kStreams + s];
    for (int64_t j = threadIdx.x; j < d; j += blockDim.x) {
        const float v = load_as_f32(y, t * d + j);
#pragma unroll
        for (int s = 0; s < kStreams; ++s) {
            store_from_f32(xr, s * d + j, fmaf(wi[s], v, load_as_f32(xr, s * d + j)));
            const float kept = load_as_f32(xr, s * d + j);  // the stored (rounded) value, as the next mix reads it
            ssq[s] = fmaf(kept, kept, ssq[s]);
        }
    }
#pragma unroll
    for (int s = 0; s < kStreams; ++s) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq[s] += __shfl_xor_sync(0xffffffffu, ssq[s], o);
        if ((threadIdx.x & 31) == 0) red[s][threadIdx.x >> 5] = ssq[s];
    }
    __syncthreads();
    if (threadIdx.x < kStreams) {
        float sum = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sum += red[threadIdx.x][w];
        inv[t * kStreams + threadIdx.x] = 1.0f / sqrtf(sum / (float)d + eps);
    }
}

// ---- up ------------------------------------------------------------------------------------------------------------

// Chunk-major W_up [N = 4 d, r] (32-code chunk c of row n at word (c N + n) * cw, group g's scale / min at [g N + n]) ->
// row-major [N, Kp] with Kp >= r: the chunks and groups past r are zero codes, zero scale, zero min.  Row
// rb * 128 + q * 32 + l of the result is W_up's row s d + j with s = l & 3, j = rb * 32 + q * 8 + (l >> 2): the order in
// which the up mix's epilogue wants the rows in tensor-memory lanes (TcHcUp).
__device__ inline int64_t up_source_row(int64_t row, int64_t d) {
    const int64_t rb = row >> 7, q = (row >> 5) & 3, l = row & 31;
    return (l & 3) * d + rb * 32 + q * 8 + (l >> 2);
}
__global__ void __launch_bounds__(256) hc_unchunk_up_kernel(const uint8_t *__restrict__ q, const uint16_t *__restrict__ scale,
                                                            const uint16_t *__restrict__ minv, int64_t d, int64_t r, int64_t Kp, int64_t G,
                                                            int bits, uint32_t *__restrict__ qo, uint16_t *__restrict__ so,
                                                            uint16_t *__restrict__ mo) {
    const int64_t N = kStreams * d;
    const int64_t cv = bits / 4, chunks = r / kChunk, chunks_p = Kp / kChunk, groups = r / G, groups_p = Kp / G;  // cv: 16-byte pieces a chunk
    const int64_t stride = (int64_t)gridDim.x * blockDim.x, first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint4 *qi = reinterpret_cast<const uint4 *>(q);
    uint4 *qv = reinterpret_cast<uint4 *>(qo);
    for (int64_t i = first; i < N * chunks_p * cv; i += stride) {
        const int64_t w = i % cv, nc = i / cv, c = nc % chunks_p, n = up_source_row(nc / chunks_p, d);
        qv[i] = c < chunks ? __ldg(qi + (c * N + n) * cv + w) : make_uint4(0u, 0u, 0u, 0u);
    }
    for (int64_t i = first; i < N * groups_p; i += stride) {
        const int64_t g = i % groups_p, n = up_source_row(i / groups_p, d);
        so[i] = g < groups ? scale[g * N + n] : (uint16_t)0, mo[i] = g < groups ? minv[g * N + n] : (uint16_t)0;
    }
}

// h [M, r] FP32 -> F16, tile-blocked in the rows' own order (a dense projection's operand), r padded to Kp with zeros.
template <int BITS>
__global__ void __launch_bounds__(256) hc_stage_h_kernel(const float *__restrict__ h, int64_t M, int64_t r, int64_t Kp,
                                                         unsigned char *__restrict__ hs) {
    const int64_t chunks_p = Kp / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * chunks_p; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / chunks_p;
        const int kk = (int)(i % chunks_p);
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if ((int64_t)kk * 8 < r) load8(h + t * r, (int64_t)kk * 8, f);
        *reinterpret_cast<uint4 *>(hs + tiled_offset(M, kk >> 3, t, (int)(t & 7), kk & 7)) = f16_chunk<BITS>(f);
    }
}

// ---- hosts ---------------------------------------------------------------------------------------------------------

int check_shape(const char *fn, int64_t T, int64_t H, int64_t d, const SxbQView *w, int act) {
    SXB_CHECK(H == kStreams, fn, ": H = ", H, " streams, only ", kStreams, " is supported");
    SXB_CHECK(T >= 1 && T <= 65535, fn, ": T = ", T, " tokens, expected 1..65535");
    SXB_CHECK(d >= 128 && d <= (1 << 20) && d % 128 == 0, fn, ": d = ", d, ", the tensor-core mix needs a multiple of 128 up to ", 1 << 20);
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SXB_CHECK(w != nullptr && w->q != nullptr && w->scale != nullptr && w->minv != nullptr, fn, ": null weight pointer");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->K >= w->G && w->K % w->G == 0, fn, ": K = ", w->K, " must be a positive multiple of group size ", w->G);
    SXB_CHECK(aligned16(w->q), fn, ": code array ", (const void *)w->q, " must be 16-byte aligned");
    return SXB_OK;
}

// Parts of the down mix's workspace, in bytes from its start; the grouping workspace comes first, so that
// sxb_check_grouped_status reads the caller's pointer as it is.
struct DownWs {
    size_t route, route_bytes, wq, wscale, wmin, xs, partial, total;
};
DownWs down_ws(int64_t T, int64_t d, int64_t R, int bits, int64_t G) {
    const int64_t Rp = up16(R), S = T * kStreams;
    DownWs L{};
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t o = at; at += al256(bytes); return o; };
    L.route_bytes = (size_t)route_words(S, 1, kStreams).total * 4;
    L.route = take(L.route_bytes);
    L.wq = take((size_t)kStreams * Rp * d * bits / 8), L.wscale = take((size_t)kStreams * Rp * (d / G) * 2), L.wmin = take((size_t)kStreams * Rp * (d / G) * 2);
    L.xs = take((size_t)S * d * 2), L.partial = take((size_t)S * Rp * 4);
    L.total = at;
    return L;
}

template <int BITS>
int mix_down_tc(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h, float *w_in,
                float *inv, void *ws, size_t ws_bytes, int act, int inv_ready, sxb_stream_t stream) {
    const char *fn = "hc_mix_down_wmma";
    if (int rc = check_shape(fn, T, H, d, w, act)) return rc;
    SXB_CHECK(d % w->G == 0, fn, ": d = ", d, " not a multiple of group size ", w->G, " (each stream's K range must start a group)");
    SXB_CHECK(x != nullptr && h != nullptr && inv != nullptr && ws != nullptr, fn, ": null pointer (x=", x, ", h=", (const void *)h,
              ", inv=", (const void *)inv, ", ws=", ws, ")");
    SXB_CHECK((inject != 0) == (w_in != nullptr), fn, ": w_in must be given exactly when inject (inject=", inject, ", w_in=", (const void *)w_in, ")");
    SXB_CHECK(r >= 1 && r <= kMaxRank, fn, ": r = ", r, ", expected 1..", kMaxRank);
    const int64_t R = r + (inject ? H : 0), Rp = up16(R), S = T * kStreams;
    SXB_CHECK(w->K == H * d && w->N == R, fn, ": weight [", w->N, ", ", w->K, "], expected [r", inject ? " + H" : "", " = ", R, ", H*d = ", H * d, "]");
    SXB_CHECK(aligned16(x) && reinterpret_cast<uintptr_t>(ws) % 256 == 0, fn, ": x must be 16-byte and the workspace 256-byte aligned");
    SXB_CHECK(std::isfinite(eps) && eps > 0.f, fn, ": eps must be finite and > 0, got ", eps);
    const DownWs L = down_ws(T, d, R, BITS, w->G);
    SXB_CHECK(ws_bytes >= L.total, fn, ": workspace of ", ws_bytes, " bytes, needs ", L.total);
    auto *base = static_cast<unsigned char *>(ws);
    auto st = static_cast<cudaStream_t>(stream);
    auto *partial = reinterpret_cast<float *>(base + L.partial);
    SxbQView stacked{base + L.wq, reinterpret_cast<uint16_t *>(base + L.wscale), reinterpret_cast<uint16_t *>(base + L.wmin), kStreams * Rp, d, w->G};

    const int64_t stack_vecs = kStreams * Rp * d * BITS / 128;
    hc_stack_down_kernel<<<(unsigned)std::min<int64_t>((stack_vecs + 255) / 256, (int64_t)sm_count() * 8), 256, 0, st>>>(
        w->q, w->scale, w->minv, R, Rp, d, w->G, BITS, reinterpret_cast<uint32_t *>(base + L.wq), reinterpret_cast<uint16_t *>(base + L.wscale),
        reinterpret_cast<uint16_t *>(base + L.wmin));
    SXB_CHECK_LAUNCH(fn, " restacking the weight, R=", R, " d=", d);
    if (int rc = regular_routes(fn, T, kStreams, base + L.route, L.route_bytes, stream)) return rc;
    const unsigned stage_blocks = (unsigned)std::min<int64_t>((S + 7) / 8, (int64_t)sm_count() * 8);
    if (act == SXB_ACT_F32)
        hc_stage_down_kernel<float, BITS><<<stage_blocks, 256, 0, st>>>(static_cast<const float *>(x), T, d, eps, inv_ready == 0, inv, base + L.xs);
    else
        hc_stage_down_kernel<uint16_t, BITS><<<stage_blocks, 256, 0, st>>>(static_cast<const uint16_t *>(x), T, d, eps, inv_ready == 0, inv, base + L.xs);
    SXB_CHECK_LAUNCH(fn, " staging the streams, T=", T, " d=", d);
    if (int rc = tc_partial_grouped<BITS>(fn, base + L.xs, &stacked, kStreams, base + L.route, L.route_bytes, S, 1, partial, SXB_ACT_F16_TILED,
                                          BITS == 4 ? 3 : 4, false, stream))
        return rc;
    hc_finish_down_kernel<<<(unsigned)((T * R + 255) / 256), 256, 0, st>>>(partial, inv, T, R, Rp, r, h, w_in);
    SXB_CHECK_LAUNCH(fn, " Q", BITS, " ", act_name(act), " T=", T, " R=", R, " d=", d, " G=", w->G);
    return SXB_OK;
}

struct UpWs {
    size_t wq, wscale, wmin, hs, total;
};
UpWs up_ws(int64_t T, int64_t d, int64_t r, int bits, int64_t G) {
    const int64_t Kp = up128(r), N = kStreams * d;
    UpWs L{};
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t o = at; at += al256(bytes); return o; };
    L.wq = take((size_t)N * Kp * bits / 8), L.wscale = take((size_t)N * (Kp / G) * 2), L.wmin = take((size_t)N * (Kp / G) * 2);
    L.hs = take((size_t)T * Kp * 2);
    L.total = at;
    return L;
}

template <int BITS>
int mix_up_tc(const float *h, const SxbQView *w, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d,
              void *u, void *ws, size_t ws_bytes, int act, sxb_stream_t stream) {
    const char *fn = "hc_mix_up_wmma";
    if (int rc = check_shape(fn, T, H, d, w, act)) return rc;
    SXB_CHECK(h != nullptr && x != nullptr && norm_w != nullptr && inv != nullptr && u != nullptr && ws != nullptr, fn, ": null pointer (h=",
              (const void *)h, ", x=", x, ", norm_w=", (const void *)norm_w, ", inv=", (const void *)inv, ", u=", u, ", ws=", ws, ")");
    SXB_CHECK(w->N == H * d, fn, ": W_up has ", w->N, " rows, expected H*d = ", H * d);
    SXB_CHECK(w->K >= kChunk && w->K <= kMaxRank && w->K % kChunk == 0, fn, ": W_up K (the rank r) = ", w->K, ", expected a multiple of ", kChunk,
              " up to ", kMaxRank);
    SXB_CHECK(aligned16(h) && aligned16(x) && aligned16(norm_w) && aligned16(u) && reinterpret_cast<uintptr_t>(ws) % 256 == 0, fn,
              ": h, x, norm_w and u must be 16-byte and the workspace 256-byte aligned");
    SXB_CHECK(w->K % 8 == 0, fn, ": r = ", w->K, " must be a multiple of 8");
    SXB_CHECK(apart(u, T * d * act_bytes(act), x, T * H * d * act_bytes(act)), fn, ": u overlaps the streams x");
    const int64_t r = w->K, Kp = up128(r), N = H * d;
    const UpWs L = up_ws(T, d, r, BITS, w->G);
    SXB_CHECK(ws_bytes >= L.total, fn, ": workspace of ", ws_bytes, " bytes, needs ", L.total);
    auto *base = static_cast<unsigned char *>(ws);
    auto st = static_cast<cudaStream_t>(stream);
    SxbQView rows{base + L.wq, reinterpret_cast<uint16_t *>(base + L.wscale), reinterpret_cast<uint16_t *>(base + L.wmin), N, Kp, w->G};

    const int64_t vecs = N * Kp * BITS / 128;
    hc_unchunk_up_kernel<<<(unsigned)std::min<int64_t>((vecs + 255) / 256, (int64_t)sm_count() * 8), 256, 0, st>>>(
        w->q, w->scale, w->minv, d, r, Kp, w->G, BITS, reinterpret_cast<uint32_t *>(base + L.wq), reinterpret_cast<uint16_t *>(base + L.wscale),
        reinterpret_cast<uint16_t *>(base + L.wmin));
    SXB_CHECK_LAUNCH(fn, " un-chunking the weight, N=", N, " r=", r);
    const unsigned stage_blocks = (unsigned)std::min<int64_t>((T * (Kp / 8) + 255) / 256, (int64_t)sm_count() * 8);
    hc_stage_h_kernel<BITS><<<stage_blocks, 256, 0, st>>>(h, T, r, Kp, base + L.hs);
    SXB_CHECK_LAUNCH(fn, " staging h, T=", T, " r=", r);
    return tc_hc_up<BITS>(fn, base + L.hs, &rows, x, inv, norm_w, u, T, d, act == SXB_ACT_F32, stream);
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" {

size_t sxb_hc_mix_down_wmma_workspace_bytes(int64_t T, int64_t H, int64_t d, int64_t R, int bits, int64_t G) {
    if (T < 1 || T > 65535 || H != kStreams || d < 128 || d % 128 != 0 || R < 1 || R > kMaxRank + kStreams || (bits != 4 && bits != 8) ||
        (G != 32 && G != 64 && G != 128)) {
        last_error() = cat("hc_mix_down_wmma_workspace_bytes: T = ", T, ", H = ", H, ", d = ", d, ", R = ", R, ", bits = ", bits, ", G = ", G);
        return 0;
    }
    return down_ws(T, d, R, bits, G).total;
}
int sxb_hc_mix_down_wmma_q4(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                            float *w_in, float *inv, void *ws, size_t ws_bytes, int act, int inv_ready, sxb_stream_t stream) {
    return mix_down_tc<4>(x, w, T, H, d, r, inject, eps, h, w_in, inv, ws, ws_bytes, act, inv_ready, stream);
}
int sxb_hc_mix_down_wmma_q8(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                            float *w_in, float *inv, void *ws, size_t ws_bytes, int act, int inv_ready, sxb_stream_t stream) {
    return mix_down_tc<8>(x, w, T, H, d, r, inject, eps, h, w_in, inv, ws, ws_bytes, act, inv_ready, stream);
}

int sxb_hc_inject_inv(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, float eps, float *inv, int act,
                      sxb_stream_t stream) {
    const char *fn = "hc_inject_inv";
    SXB_CHECK(H == kStreams, fn, ": H = ", H, " streams, only ", kStreams, " is supported");
    SXB_CHECK(T >= 1 && T <= 0x7fffffff && d >= 1 && d <= (1 << 20), fn, ": T = ", T, ", d = ", d);
    SXB_CHECK(x != nullptr && w_in != nullptr && y != nullptr && inv != nullptr, fn, ": null pointer (x=", x, ", w_in=", (const void *)w_in,
              ", y=", y, ", inv=", (const void *)inv, ")");
    SXB_CHECK(std::isfinite(eps) && eps > 0.f, fn, ": eps must be finite and > 0, got ", eps);
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SXB_CHECK(apart(x, T * H * d * act_bytes(act), y, T * d * act_bytes(act)), fn, ": y overlaps the streams x");
    auto st = static_cast<cudaStream_t>(stream);
    if (act == SXB_ACT_F32)
        hc_inject_inv_kernel<float><<<(unsigned)T, 256, 0, st>>>(static_cast<float *>(x), w_in, static_cast<const float *>(y), d, eps, inv);
    else
        hc_inject_inv_kernel<uint16_t><<<(unsigned)T, 256, 0, st>>>(static_cast<uint16_t *>(x), w_in, static_cast<const uint16_t *>(y), d, eps, inv);
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), " T=", T, " d=", d);
    return SXB_OK;
}

size_t sxb_hc_mix_up_wmma_workspace_bytes(int64_t T, int64_t H, int64_t d, int64_t r, int bits, int64_t G) {
    if (T < 1 || T > 65535 || H != kStreams || d < 128 || d % 128 != 0 || r < kChunk || r > kMaxRank || r % kChunk != 0 ||
        (bits != 4 && bits != 8) || (G != 32 && G != 64 && G != 128)) {
        last_error() = cat("hc_mix_up_wmma_workspace_bytes: T = ", T, ", H = ", H, ", d = ", d, ", r = ", r, ", bits = ", bits, ", G = ", G);
        return 0;
    }
    return up_ws(T, d, r, bits, G).total;
}
int sxb_hc_mix_up_wmma_q4(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                          int64_t d, void *u, void *ws, size_t ws_bytes, int act, sxb_stream_t stream) {
    return mix_up_tc<4>(h, w_up, x, norm_w, inv, T, H, d, u, ws, ws_bytes, act, stream);
}
int sxb_hc_mix_up_wmma_q8(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                          int64_t d, void *u, void *ws, size_t ws_bytes, int act, sxb_stream_t stream) {
    return mix_up_tc<8>(h, w_up, x, norm_w, inv, T, H, d, u, ws, ws_bytes, act, stream);
}

}  // extern "C"
