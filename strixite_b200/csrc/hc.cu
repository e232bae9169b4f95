// The hyper-connection mix that produces the MoE block's input (kernels/hc.hpp:36-50, call site
// runtime/qwen4exp.cpp:2801-2831, 3144): from the H = 4 residual streams X [T, H*d]
//   hc_mix_down   h [T, r] = silu(a / H) and w_in [T, H] = 2 sigmoid(a / H), a = sum_s inv_s * (W'_s . X_s) over the rows of
//                 the folded, quantized down weight W' [r (+ H), H*d]; inv [T, H] = 1 / sqrt(mean(X_s^2) + eps)
//   hc_mix_up     u [T, d] = (1/H) sum_s sigmoid(W_up[s*d + j] . h) * X_s[j] * inv_s * (1 + norm_w[s*d + j]), W_up chunk-major
// Everything inside is FP32 (kernels/hc.hpp:8-11); u is rounded once to the activation dtype.  A quantized row's dot with
// a 32-code chunk is scale * sum(x * code) + min * sum(x) (kernels/hc.hip:117-123, 206-211): the weights are never
// rounded to a dequantized value.
//
// Both are small-matrix, many-launch kernels (a few MB of weights, ~97 mixes per decoded token upstream): what matters is
// that the weight matrix is read once per group of tokens and that enough CTAs exist to cover the SMs at T = 1..64.
//   down: a warp owns RW weight rows and TT tokens; its lanes take the 32-code chunks of the row in turn (a chunk lies in
//         one stream since d % 32 == 0), keep per-stream partial dots in registers, and meet by shuffles.  Each chunk's
//         sum(x) and sum(x^2) are the same for every row: computed once per CTA into shared memory.
//   up:   a thread owns one row s*d + j of W_up (consecutive threads' rows are adjacent in the chunk-major layout, so a
//         warp's 16-byte loads are one contiguous run), dots it with the h of MT tokens held in shared memory, and the
//         H streams of a column meet in shared memory.

#include "experts.cuh"

#include <algorithm>
#include <cmath>

namespace sxb {
namespace {

constexpr int kHcThreads = 256;
constexpr int kStreams = 4;
constexpr int kChunk = 32;  // codes per chunk: 16 bytes of Q4, 32 of Q8
constexpr int64_t kMaxRank = 1024;

// 32 activations of one chunk as FP32.
__device__ inline void load_chunk_x(const float *x, float (&v)[kChunk]) {
#pragma unroll
    for (int i = 0; i < kChunk / 4; ++i) {
        const float4 f = __ldg(reinterpret_cast<const float4 *>(x) + i);
        v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
    }
}
__device__ inline void load_chunk_x(const uint16_t *x, float (&v)[kChunk]) {
#pragma unroll
    for (int i = 0; i < kChunk / 8; ++i) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(x) + i);
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) v[8 * i + 2 * j] = __uint_as_float(w4[j] << 16), v[8 * i + 2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
    }
}
// The 32 codes of a chunk as FP32 (Q4: low nibble = even code).
template <int BITS>
__device__ inline void load_chunk_codes(const uint8_t *p, float (&c)[kChunk]) {
    constexpr int WORDS = BITS;  // 4 words of Q4, 8 of Q8
    uint32_t w[WORDS];
#pragma unroll
    for (int i = 0; i < WORDS / 4; ++i) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(p) + i);
        w[4 * i] = u.x, w[4 * i + 1] = u.y, w[4 * i + 2] = u.z, w[4 * i + 3] = u.w;
    }
    constexpr int per = 32 / BITS;
#pragma unroll
    for (int i = 0; i < kChunk; ++i) c[i] = (float)((w[i / per] >> (BITS * (i % per))) & ((1u << BITS) - 1u));
}
__device__ inline float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }

// hc_mix_down.  grid = (row groups, token groups); a warp: rows n0 .. n0 + RW - 1, tokens t0 .. t0 + TT - 1.
template <typename T, int BITS, int RW, int TT>
__global__ void __launch_bounds__(kHcThreads) hc_down_kernel(const T *__restrict__ x, const uint8_t *__restrict__ q,
                                                             const uint16_t *__restrict__ scale, const uint16_t *__restrict__ minv, int64_t R,
                                                             int64_t K, int64_t G, int64_t d, int r, float eps, int64_t Tn,
                                                             float *__restrict__ h, float *__restrict__ w_in, float *__restrict__ inv) {
    extern __shared__ float2 sums[];  // [TT][K / 32]: each chunk's sum(x) and sum(x^2)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kHcThreads / 32;
    const int64_t nc = K / kChunk, t0 = (int64_t)blockIdx.y * TT;
    const int nt = (int)min((int64_t)TT, Tn - t0);
    for (int64_t i = threadIdx.x; i < nt * nc; i += kHcThreads) {
        const int tt = (int)(i / nc);
        const int64_t c = i % nc;
        float xv[kChunk];
        load_chunk_x(x + (t0 + tt) * K + c * kChunk, xv);
        float s = 0.f, sq = 0.f;
#pragma unroll
        for (int k = 0; k < kChunk; ++k) s += xv[k], sq = fmaf(xv[k], xv[k], sq);
        sums[tt * nc + c] = make_float2(s, sq);
    }
    __syncthreads();
    const int64_t n0 = ((int64_t)blockIdx.x * warps + warp) * RW;
    if (n0 >= R) return;
    float dot[RW][TT][kStreams], sq[TT][kStreams];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
        for (int s = 0; s < kStreams; ++s) {
            sq[tt][s] = 0.f;
#pragma unroll
            for (int rw = 0; rw < RW; ++rw) dot[rw][tt][s] = 0.f;
        }
    const int64_t row_bytes = K * BITS / 8, groups = K / G;
    for (int64_t c = lane; c < nc; c += 32) {
        const int g = (int)(c * kChunk / d);  // the chunk's stream
        float code[RW][kChunk], sc[RW], mn[RW];
#pragma unroll
        for (int rw = 0; rw < RW; ++rw) {
            const int64_t n = min(n0 + rw, R - 1);  // a row past the end repeats the last one; its sums are dropped
            load_chunk_codes<BITS>(q + n * row_bytes + c * (kChunk * BITS / 8), code[rw]);
            sc[rw] = bf16_bits_to_f32(__ldg(scale + n * groups + c * kChunk / G));
            mn[rw] = bf16_bits_to_f32(__ldg(minv + n * groups + c * kChunk / G));
        }
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            if (tt >= nt) break;
            float xv[kChunk];
            load_chunk_x(x + (t0 + tt) * K + c * kChunk, xv);
            const float2 ss = sums[tt * nc + c];
#pragma unroll
            for (int rw = 0; rw < RW; ++rw) {
                float dsum = 0.f;
#pragma unroll
                for (int k = 0; k < kChunk; ++k) dsum = fmaf(xv[k], code[rw][k], dsum);
                const float pv = fmaf(sc[rw], dsum, mn[rw] * ss.x);
#pragma unroll
                for (int s = 0; s < kStreams; ++s)  // static indices keep the sums in registers
                    if (s == g) dot[rw][tt][s] += pv;
            }
#pragma unroll
            for (int s = 0; s < kStreams; ++s)
                if (s == g) sq[tt][s] += ss.y;
        }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
        for (int s = 0; s < kStreams; ++s) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sq[tt][s] += __shfl_xor_sync(0xffffffffu, sq[tt][s], off);
#pragma unroll
            for (int rw = 0; rw < RW; ++rw)
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) dot[rw][tt][s] += __shfl_xor_sync(0xffffffffu, dot[rw][tt][s], off);
        }
    if (lane != 0) return;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        if (tt >= nt) break;
        const int64_t t = t0 + tt;
        float iv[kStreams];
#pragma unroll
        for (int s = 0; s < kStreams; ++s) iv[s] = 1.0f / sqrtf(sq[tt][s] / (float)d + eps);
#pragma unroll
        for (int rw = 0; rw < RW; ++rw) {
            const int64_t n = n0 + rw;
            if (n >= R) break;
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < kStreams; ++s) a = fmaf(iv[s], dot[rw][tt][s], a);
            const float z = a / (float)kStreams;
            if (n < r) h[t * r + n] = z * sigmoid_f32(z);
            else w_in[t * kStreams + (n - r)] = 2.0f * sigmoid_f32(z);
        }
        if (n0 == 0)
#pragma unroll
            for (int s = 0; s < kStreams; ++s) inv[t * kStreams + s] = iv[s];
    }
}

// hc_mix_up.  grid = (d / 64, token groups of MT); thread (s, jl) owns row s*d + j of W_up.
constexpr int kUpCols = kHcThreads / kStreams;  // 64 output columns per CTA

template <typename T, int BITS, int MT>
__global__ void __launch_bounds__(kHcThreads) hc_up_kernel(const float *__restrict__ h, const uint8_t *__restrict__ q,
                                                           const uint16_t *__restrict__ scale, const uint16_t *__restrict__ minv, int64_t G,
                                                           const T *__restrict__ x, const float *__restrict__ norm_w,
                                                           const float *__restrict__ inv, int64_t d, int r, int64_t Tn, T *__restrict__ u) {
    extern __shared__ float up_smem[];  // hs [MT][r], hsum [MT][r / 32], part [MT][H][64]
    float *hs = up_smem, *hsum = hs + (size_t)MT * r, *part = hsum + (size_t)MT * (r / kChunk);
    const int64_t t0 = (int64_t)blockIdx.y * MT, N = kStreams * d;
    const int nt = (int)min((int64_t)MT, Tn - t0), chunks = r / kChunk;
    for (int i = threadIdx.x; i < nt * r; i += kHcThreads) hs[i] = h[t0 * r + i];
    __syncthreads();
    for (int i = threadIdx.x; i < nt * chunks; i += kHcThreads) {
        float s = 0.f;
        for (int k = 0; k < kChunk; ++k) s += hs[(i / chunks) * r + (i % chunks) * kChunk + k];
        hsum[i] = s;
    }
    __syncthreads();
    const int s = threadIdx.x / kUpCols, jl = threadIdx.x % kUpCols;
    const int64_t j = (int64_t)blockIdx.x * kUpCols + jl;
    if (j < d) {
        const int64_t row = s * d + j;
        float acc[MT];
#pragma unroll
        for (int tt = 0; tt < MT; ++tt) acc[tt] = 0.f;
        for (int c = 0; c < chunks; ++c) {
            float code[kChunk];
            load_chunk_codes<BITS>(q + ((int64_t)c * N + row) * (kChunk * BITS / 8), code);
            const int64_t gi = (int64_t)(c * kChunk / G) * N + row;
            const float sc = bf16_bits_to_f32(__ldg(scale + gi)), mn = bf16_bits_to_f32(__ldg(minv + gi));
#pragma unroll
            for (int tt = 0; tt < MT; ++tt) {
                if (tt >= nt) break;
                const float *hv = hs + tt * r + c * kChunk;
                float dsum = 0.f;
#pragma unroll
                for (int k = 0; k < kChunk; ++k) dsum = fmaf(hv[k], code[k], dsum);
                acc[tt] = fmaf(sc, dsum, fmaf(mn, hsum[tt * chunks + c], acc[tt]));
            }
        }
        const float nw = 1.0f + norm_w[row];
#pragma unroll
        for (int tt = 0; tt < MT; ++tt) {
            if (tt >= nt) break;
            const int64_t t = t0 + tt;
            part[(tt * kStreams + s) * kUpCols + jl] = sigmoid_f32(acc[tt]) * (load_as_f32(x, t * N + row) * inv[t * kStreams + s] * nw);
        }
    }
    __syncthreads();
    if (s == 0 && j < d)
        for (int tt = 0; tt < nt; ++tt) {
            float sum = 0.f;
#pragma unroll
            for (int k = 0; k < kStreams; ++k) sum += part[(tt * kStreams + k) * kUpCols + jl];
            store_from_f32(u, (t0 + tt) * d + j, sum / (float)kStreams);
        }
}

// Row-major Q4 / Q8 -> chunk-major (formats/q4.hpp:41-55): 32-code chunk c of row n at q[(c * N + n) * chunk bytes], group
// g's scale / min at [g * N + n].
__global__ void __launch_bounds__(256) chunk_major_kernel(const uint8_t *__restrict__ q, const uint16_t *__restrict__ scale,
                                                          const uint16_t *__restrict__ minv, int64_t N, int64_t K, int64_t G, int chunk_bytes,
                                                          uint8_t *__restrict__ qo, uint16_t *__restrict__ so, uint16_t *__restrict__ mo) {
    const int64_t chunks = K / kChunk, groups = K / G, words = chunk_bytes / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N * chunks * words; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t w = i % words, nc = i / words, c = nc % chunks, n = nc / chunks;
        reinterpret_cast<uint32_t *>(qo)[(c * N + n) * words + w] = reinterpret_cast<const uint32_t *>(q)[(n * chunks + c) * words + w];
    }
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N * groups; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = i % groups, n = i / groups;
        so[g * N + n] = scale[i], mo[g * N + n] = minv[i];
    }
}

int check_hc_shape(const char *fn, int64_t T, int64_t H, int64_t d) {
    SXB_CHECK(H == kStreams, fn, ": H = ", H, " streams, only ", kStreams, " is supported");
    SXB_CHECK(T >= 1 && T <= 65535, fn, ": T = ", T, " tokens, expected 1..65535");
    SXB_CHECK(d >= kChunk && d <= (1 << 20) && d % kChunk == 0, fn, ": d = ", d, ", expected a multiple of ", kChunk, " up to ", 1 << 20);
    return SXB_OK;
}
int check_hc_weight(const char *fn, const SxbQView *w) {
    SXB_CHECK(w != nullptr && w->q != nullptr && w->scale != nullptr && w->minv != nullptr, fn, ": null weight pointer");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->K >= w->G && w->K % w->G == 0, fn, ": K = ", w->K, " must be a positive multiple of group size ", w->G);
    SXB_CHECK(aligned16(w->q), fn, ": code array ", (const void *)w->q, " must be 16-byte aligned for vector loads");
    return SXB_OK;
}

template <int BITS>
int mix_down(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h, float *w_in,
             float *inv, int act, sxb_stream_t stream) {
    const char *fn = "hc_mix_down";
    if (int rc = check_hc_shape(fn, T, H, d)) return rc;
    if (int rc = check_hc_weight(fn, w)) return rc;
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SXB_CHECK(x != nullptr && h != nullptr && inv != nullptr, fn, ": null pointer (x=", x, ", h=", (const void *)h, ", inv=", (const void *)inv, ")");
    SXB_CHECK((inject != 0) == (w_in != nullptr), fn, ": w_in must be given exactly when inject (inject=", inject, ", w_in=", (const void *)w_in, ")");
    SXB_CHECK(r >= 1 && r <= kMaxRank, fn, ": r = ", r, ", expected 1..", kMaxRank);
    SXB_CHECK(w->K == H * d, fn, ": weight K = ", w->K, " != H*d = ", H * d);
    const int64_t R = r + (inject ? H : 0);
    SXB_CHECK(w->N == R, fn, ": weight has ", w->N, " rows, expected r", inject ? " + H" : "", " = ", R);
    SXB_CHECK(aligned16(x), fn, ": x ", x, " must be 16-byte aligned");
    SXB_CHECK(std::isfinite(eps) && eps > 0.f, fn, ": eps must be finite and > 0, got ", eps);
    // Tokens per warp: as many as keeps at least one CTA per SM in the grid (every token group re-reads the weight from L2).
    const int64_t row_groups1 = (R + 7) / 8;
    int TT = 4;
    while (TT > 1 && row_groups1 * ((T + TT - 1) / TT) < sm_count()) TT >>= 1;
    const size_t smem = (size_t)TT * (size_t)(w->K / kChunk) * sizeof(float2);
    SXB_CHECK(smem <= 160 * 1024, fn, ": H*d = ", w->K, " needs ", smem, " bytes of shared memory for its chunk sums");
    auto st = static_cast<cudaStream_t>(stream);
    // two rows a warp once the grid is large anyway (each activation load then meets two rows)
    const bool two = (R + 15) / 16 * ((T + TT - 1) / TT) >= 2 * sm_count();
#define SXB_HC_DOWN(TYPE, RW, TTV)                                                                                                     \
    do {                                                                                                                               \
        auto kern = hc_down_kernel<TYPE, BITS, RW, TTV>;                                                                               \
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory"); \
        const dim3 grid((unsigned)((R + 8 * RW - 1) / (8 * RW)), (unsigned)((T + TTV - 1) / TTV));                                     \
        kern<<<grid, kHcThreads, smem, st>>>(static_cast<const TYPE *>(x), w->q, w->scale, w->minv, R, w->K, w->G, d, (int)r, eps, T, h, \
                                             w_in, inv);                                                                               \
    } while (0)
#define SXB_HC_DOWN_T(TYPE)                             \
    do {                                                \
        if (TT == 4 && two) SXB_HC_DOWN(TYPE, 2, 4);    \
        else if (TT == 4) SXB_HC_DOWN(TYPE, 1, 4);      \
        else if (TT == 2) SXB_HC_DOWN(TYPE, 1, 2);      \
        else SXB_HC_DOWN(TYPE, 1, 1);                   \
    } while (0)
    if (act == SXB_ACT_F32) SXB_HC_DOWN_T(float);
    else SXB_HC_DOWN_T(uint16_t);
#undef SXB_HC_DOWN_T
#undef SXB_HC_DOWN
    SXB_CHECK_LAUNCH(fn, " Q", BITS, " ", act_name(act), " T=", T, " R=", R, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

template <int BITS>
int mix_up(const float *h, const SxbQView *w, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d,
           void *u, int act, sxb_stream_t stream) {
    const char *fn = "hc_mix_up";
    if (int rc = check_hc_shape(fn, T, H, d)) return rc;
    if (int rc = check_hc_weight(fn, w)) return rc;
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SXB_CHECK(h != nullptr && x != nullptr && norm_w != nullptr && inv != nullptr && u != nullptr, fn, ": null pointer (h=", (const void *)h,
              ", x=", x, ", norm_w=", (const void *)norm_w, ", inv=", (const void *)inv, ", u=", u, ")");
    SXB_CHECK(w->N == H * d, fn, ": W_up has ", w->N, " rows, expected H*d = ", H * d);
    SXB_CHECK(w->K >= kChunk && w->K <= kMaxRank && w->K % kChunk == 0, fn, ": W_up K (the rank r) = ", w->K, ", expected a multiple of ",
              kChunk, " up to ", kMaxRank);
    SXB_CHECK(apart(u, T * d * act_bytes(act), x, T * H * d * act_bytes(act)), fn, ": u overlaps the streams x");
    const int64_t r = w->K, col_groups = (d + kUpCols - 1) / kUpCols;
    int MT = 8;
    while (MT > 1 && (col_groups * ((T + MT - 1) / MT) < sm_count() || MT > T)) MT >>= 1;
    const size_t smem = ((size_t)MT * r + (size_t)MT * (r / kChunk) + (size_t)MT * kStreams * kUpCols) * sizeof(float);
    auto st = static_cast<cudaStream_t>(stream);
#define SXB_HC_UP(TYPE, MTV)                                                                                                           \
    do {                                                                                                                               \
        auto kern = hc_up_kernel<TYPE, BITS, MTV>;                                                                                     \
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory"); \
        const dim3 grid((unsigned)col_groups, (unsigned)((T + MTV - 1) / MTV));                                                        \
        kern<<<grid, kHcThreads, smem, st>>>(h, w->q, w->scale, w->minv, w->G, static_cast<const TYPE *>(x), norm_w, inv, d, (int)r, T,    \
                                             static_cast<TYPE *>(u));                                                                  \
    } while (0)
#define SXB_HC_UP_T(TYPE)                    \
    do {                                     \
        if (MT == 8) SXB_HC_UP(TYPE, 8);     \
        else if (MT == 4) SXB_HC_UP(TYPE, 4);\
        else if (MT == 2) SXB_HC_UP(TYPE, 2);\
        else SXB_HC_UP(TYPE, 1);             \
    } while (0)
    if (act == SXB_ACT_F32) SXB_HC_UP_T(float);
    else SXB_HC_UP_T(uint16_t);
#undef SXB_HC_UP_T
#undef SXB_HC_UP
    SXB_CHECK_LAUNCH(fn, " Q", BITS, " ", act_name(act), " T=", T, " d=", d, " r=", r, " G=", w->G, " MT=", MT);
    return SXB_OK;
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" {

int sxb_hc_mix_down_q4(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                       float *w_in, float *inv, int act, sxb_stream_t stream) {
    return mix_down<4>(x, w, T, H, d, r, inject, eps, h, w_in, inv, act, stream);
}
int sxb_hc_mix_down_q8(const void *x, const SxbQView *w, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                       float *w_in, float *inv, int act, sxb_stream_t stream) {
    return mix_down<8>(x, w, T, H, d, r, inject, eps, h, w_in, inv, act, stream);
}
int sxb_hc_mix_up_q4(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                     int64_t d, void *u, int act, sxb_stream_t stream) {
    return mix_up<4>(h, w_up, x, norm_w, inv, T, H, d, u, act, stream);
}
int sxb_hc_mix_up_q8(const float *h, const SxbQView *w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H,
                     int64_t d, void *u, int act, sxb_stream_t stream) {
    return mix_up<8>(h, w_up, x, norm_w, inv, T, H, d, u, act, stream);
}

int sxb_to_chunk_major(const SxbQView *w, int bits, uint8_t *q, uint16_t *scale, uint16_t *minv, sxb_stream_t stream) {
    const char *fn = "to_chunk_major";
    if (int rc = check_hc_weight(fn, w)) return rc;
    SXB_CHECK(bits == 4 || bits == 8, fn, ": ", bits, "-bit codes unsupported (4 or 8)");
    SXB_CHECK(q != nullptr && scale != nullptr && minv != nullptr, fn, ": null output pointer");
    SXB_CHECK(w->N >= 1 && w->K % kChunk == 0, fn, ": chunk-major needs K % 32 == 0 (32-code chunks), got K = ", w->K);
    SXB_CHECK(reinterpret_cast<uintptr_t>(q) % 16 == 0, fn, ": output codes must be 16-byte aligned");
    const int64_t words = w->N * (w->K / kChunk) * (bits == 4 ? 4 : 8);
    const unsigned blocks = (unsigned)std::min<int64_t>((words + 255) / 256, (int64_t)sm_count() * 8);
    chunk_major_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(w->q, w->scale, w->minv, w->N, w->K, w->G, bits == 4 ? 16 : 32, q,
                                                                             scale, minv);
    SXB_CHECK_LAUNCH(fn, " N=", w->N, " K=", w->K, " G=", w->G, " bits=", bits);
    return SXB_OK;
}

}  // extern "C"
