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
//   down: a CTA owns a group of weight rows and up to four tokens, whose streams it holds in shared memory; its sixteen warps
//         take (row, eighth of the row) items, an eighth lying in one stream, and the parts meet in shared memory.
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

__device__ inline float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }
// 16 bytes of activations as FP32: four (FP32) or eight (BF16) values.
__device__ inline void unpack16(const uint4 &u, float (&f)[4], const float *) {
    f[0] = __uint_as_float(u.x), f[1] = __uint_as_float(u.y), f[2] = __uint_as_float(u.z), f[3] = __uint_as_float(u.w);
}
__device__ inline void unpack16(const uint4 &u, float (&f)[8], const uint16_t *) {
    const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) f[2 * j] = __uint_as_float(w4[j] << 16), f[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
}

// Eight consecutive codes of a chunk (k = 8 j .. 8 j + 7) as FP32, from the chunk's packed words.
template <int BITS>
__device__ inline void codes8(const uint32_t *w, int j, float (&c)[8]) {
    if (BITS == 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) c[i] = (float)((w[2 * j + (i >> 2)] >> (8 * (i & 3))) & 0xFFu);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) c[i] = (float)((w[j] >> (4 * i)) & 0xFu);
    }
}
template <int BITS>
__device__ inline void load_chunk_words(const uint8_t *p, uint32_t (&w)[BITS]) {
#pragma unroll
    for (int i = 0; i < BITS / 4; ++i) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(p) + i);
        w[4 * i] = u.x, w[4 * i + 1] = u.y, w[4 * i + 2] = u.z, w[4 * i + 3] = u.w;
    }
}

// hc_mix_down.  grid = (row groups of RG rows, token groups of TT); one CTA of sixteen warps an SM.
//   1. The TT tokens' streams go to shared memory once (chunk-interleaved: 16-byte piece p of chunk c of token tt at
//      ((tt * P + p) * nc + c) * 16, so that lanes with consecutive chunks read consecutive 16 bytes), and each chunk's
//      sum(x) and sum(x^2) - the same for every weight row - are computed once.
//   2. The work items are (row, eighth of the row's chunks): an eighth lies in one stream (H = 4).  The warps take items in
//      turn; a lane has only a few chunks of an item and all their loads are in flight together - with a warp walking a whole
//      row, sixteen dependent rounds of loads made this kernel 57 us at T = 16.  An item's partial dot per token goes to
//      shared memory.
//   3. One thread per (row, token) adds the parts in order, applies the per-stream inverse RMS and the activation.
constexpr int kDownThreads = 512, kParts = 8;
constexpr int kMaxRowGroup = 32;

template <typename T, int BITS, int TT>
__global__ void __launch_bounds__(kDownThreads, 1) hc_down_kernel(const T *__restrict__ x, const uint8_t *__restrict__ q,
                                                                  const uint16_t *__restrict__ scale, const uint16_t *__restrict__ minv,
                                                                  int64_t R, int64_t K, int64_t G, int64_t d, int r, float eps, int64_t Tn,
                                                                  int RG, float *__restrict__ h, float *__restrict__ w_in,
                                                                  float *__restrict__ inv) {
    constexpr int P = kChunk * (int)sizeof(T) / 16;  // 16-byte pieces of a chunk of activations: 4 (BF16) or 8 (FP32)
    constexpr int kWarps = kDownThreads / 32;
    extern __shared__ __align__(16) unsigned char down_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nc = (int)(K / kChunk);
    uint4 *xs = reinterpret_cast<uint4 *>(down_smem);                                 // [TT][P][nc]
    float2 *sums = reinterpret_cast<float2 *>(down_smem + (size_t)TT * P * nc * 16);  // [TT][nc]
    float *part = reinterpret_cast<float *>(sums + (size_t)TT * nc);                  // [RG][kParts][TT]
    float *ssq = part + (size_t)kMaxRowGroup * kParts * TT;                            // [TT][H]
    const int64_t t0 = (int64_t)blockIdx.y * TT, n0 = (int64_t)blockIdx.x * RG;
    const int nt = (int)min((int64_t)TT, Tn - t0), rows = (int)min((int64_t)RG, R - n0);
    // 1. the activations, all loads of a thread in flight at once (batches of eight)
    const int pieces_per_token = nc * P;
    for (int base = threadIdx.x; base < nt * pieces_per_token; base += 8 * kDownThreads) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * kDownThreads;
            if (i < nt * pieces_per_token) {
                const int tt = i / pieces_per_token, jj = i % pieces_per_token;
                v[j] = __ldg(reinterpret_cast<const uint4 *>(x + (t0 + tt) * K) + jj);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * kDownThreads;
            if (i < nt * pieces_per_token) {
                const int tt = i / pieces_per_token, jj = i % pieces_per_token;
                xs[(tt * P + jj % P) * nc + jj / P] = v[j];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * nc; i += kDownThreads) {
        const int tt = i / nc, c = i % nc;
        float sx = 0.f, sq = 0.f;
#pragma unroll
        for (int p = 0; p < P; ++p) {
            const uint4 u = xs[(tt * P + p) * nc + c];
            float f[16 / sizeof(T)];
            unpack16(u, f, static_cast<const T *>(nullptr));
#pragma unroll
            for (int k = 0; k < (int)(16 / sizeof(T)); ++k) sx += f[k], sq = fmaf(f[k], f[k], sq);
        }
        sums[i] = make_float2(sx, sq);
    }
    __syncthreads();
    // the sum of squares of every (token, stream): one thread each, chunks in order
    if (threadIdx.x < nt * kStreams) {
        const int tt = threadIdx.x / kStreams, st = threadIdx.x % kStreams, per = nc / kStreams;
        float sq = 0.f;
        for (int c = st * per; c < (st + 1) * per; ++c) sq += sums[tt * nc + c].y;
        ssq[threadIdx.x] = sq;
    }
    // 2. items (row, part): chunks [part * nc / 8, (part + 1) * nc / 8) of row n0 + row
    const int64_t row_bytes = K * BITS / 8, groups = K / G;
    const int per_part = nc / kParts;
    for (int item = warp; item < rows * kParts; item += kWarps) {
        const int row = item / kParts, pt = item % kParts;
        const int64_t n = n0 + row;
        float acc[TT];
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) acc[tt] = 0.f;
        // a lane's chunks of the item two at a time, both chunks' loads issued before either is used
        for (int c0 = pt * per_part + lane; c0 < (pt + 1) * per_part; c0 += 64) {
            uint32_t w[2][BITS];
            float sc[2], mn[2];
            const bool two = c0 + 32 < (pt + 1) * per_part;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = e == 0 || two ? c0 + 32 * e : c0;
                load_chunk_words<BITS>(q + n * row_bytes + (int64_t)c * (kChunk * BITS / 8), w[e]);
                sc[e] = bf16_bits_to_f32(__ldg(scale + n * groups + c * kChunk / G));
                mn[e] = bf16_bits_to_f32(__ldg(minv + n * groups + c * kChunk / G));
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (e == 1 && !two) break;
                const int c = c0 + 32 * e;
                float dsum[TT];
#pragma unroll
                for (int tt = 0; tt < TT; ++tt) dsum[tt] = 0.f;
#pragma unroll
                for (int j = 0; j < kChunk / 8; ++j) {  // eight codes at a time: converted once, met by every token
                    float cf[8];
                    codes8<BITS>(w[e], j, cf);
#pragma unroll
                    for (int tt = 0; tt < TT; ++tt) {
                        if (tt >= nt) break;
                        float f[8];
                        if constexpr (sizeof(T) == 2) {
                            unpack16(xs[(tt * P + j) * nc + c], f, static_cast<const T *>(nullptr));
                        } else {
                            float g4[4];
                            unpack16(xs[(tt * P + 2 * j) * nc + c], g4, static_cast<const T *>(nullptr));
                            f[0] = g4[0], f[1] = g4[1], f[2] = g4[2], f[3] = g4[3];
                            unpack16(xs[(tt * P + 2 * j + 1) * nc + c], g4, static_cast<const T *>(nullptr));
                            f[4] = g4[0], f[5] = g4[1], f[6] = g4[2], f[7] = g4[3];
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k) dsum[tt] = fmaf(f[k], cf[k], dsum[tt]);
                    }
                }
#pragma unroll
                for (int tt = 0; tt < TT; ++tt)
                    if (tt < nt) acc[tt] += fmaf(sc[e], dsum[tt], mn[e] * sums[tt * nc + c].x);
            }
        }
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], off);
            if (lane == 0) part[(row * kParts + pt) * TT + tt] = acc[tt];
        }
    }
    __syncthreads();
    // 3. one thread per (row, token)
    for (int i = threadIdx.x; i < rows * nt; i += kDownThreads) {
        const int row = i / nt, tt = i % nt;
        const int64_t n = n0 + row, t = t0 + tt;
        float a = 0.f;
#pragma unroll
        for (int st = 0; st < kStreams; ++st) {
            float dot = 0.f;
#pragma unroll
            for (int k = 0; k < kParts / kStreams; ++k) dot += part[(row * kParts + st * (kParts / kStreams) + k) * TT + tt];
            a = fmaf(1.0f / sqrtf(ssq[tt * kStreams + st] / (float)d + eps), dot, a);
        }
        const float z = a / (float)kStreams;
        if (n < r) h[t * r + n] = z * sigmoid_f32(z);
        else w_in[t * kStreams + (n - r)] = 2.0f * sigmoid_f32(z);
    }
    if (n0 == 0 && threadIdx.x < nt * kStreams)
        inv[(t0 + threadIdx.x / kStreams) * kStreams + threadIdx.x % kStreams] = 1.0f / sqrtf(ssq[threadIdx.x] / (float)d + eps);
}

// hc_mix_up.  grid = (d / 64, token groups of MT); thread (s, jl) owns row s*d + j of W_up.  Four chunks of packed codes are
// in flight per thread (a thread has only r / 32 chunks, and one at a time made this kernel ten rounds of load latency).
constexpr int kUpCols = kHcThreads / kStreams;  // 64 output columns per CTA
constexpr int kUpAhead = 4;

template <typename T, int BITS, int MT>
__global__ void __launch_bounds__(kHcThreads) hc_up_kernel(const float *__restrict__ h, const uint8_t *__restrict__ q,
                                                           const uint16_t *__restrict__ scale, const uint16_t *__restrict__ minv, int64_t G,
                                                           const T *__restrict__ x, const float *__restrict__ norm_w,
                                                           const float *__restrict__ inv, int64_t d, int r, int64_t Tn, T *__restrict__ u) {
    extern __shared__ float up_smem[];  // hs [MT][r], hsum [MT][r / 32], part [MT][H][64]
    float *hs = up_smem, *hsum = hs + (size_t)MT * r, *part = hsum + (size_t)MT * (r / kChunk);
    const int64_t t0 = (int64_t)blockIdx.y * MT, N = kStreams * d;
    const int nt = (int)min((int64_t)MT, Tn - t0), chunks = r / kChunk;
    const int s = threadIdx.x / kUpCols, jl = threadIdx.x % kUpCols;
    const int64_t j = (int64_t)blockIdx.x * kUpCols + jl, row = s * d + min(j, d - 1);
    // the first chunks' codes are asked for before anything else
    uint32_t wq[kUpAhead][BITS];
    float sc[kUpAhead], mn[kUpAhead];
    auto fetch = [&](int slot, int c) {
        load_chunk_words<BITS>(q + ((int64_t)c * N + row) * (kChunk * BITS / 8), wq[slot]);
        const int64_t gi = (int64_t)(c * kChunk / G) * N + row;
        sc[slot] = bf16_bits_to_f32(__ldg(scale + gi)), mn[slot] = bf16_bits_to_f32(__ldg(minv + gi));
    };
#pragma unroll
    for (int a = 0; a < kUpAhead; ++a)
        if (a < chunks) fetch(a, a);
    for (int i = threadIdx.x; i < nt * r; i += kHcThreads) hs[i] = h[t0 * r + i];
    __syncthreads();
    for (int i = threadIdx.x; i < nt * chunks; i += kHcThreads) {
        float sum = 0.f;
        for (int k = 0; k < kChunk; ++k) sum += hs[(i / chunks) * r + (i % chunks) * kChunk + k];
        hsum[i] = sum;
    }
    __syncthreads();
    float acc[MT];
#pragma unroll
    for (int tt = 0; tt < MT; ++tt) acc[tt] = 0.f;
    for (int c0 = 0; c0 < chunks; c0 += kUpAhead) {
#pragma unroll
        for (int a = 0; a < kUpAhead; ++a) {
            const int c = c0 + a;
            if (c >= chunks) break;
            float dsum[MT];
#pragma unroll
            for (int tt = 0; tt < MT; ++tt) dsum[tt] = 0.f;
#pragma unroll
            for (int jj = 0; jj < kChunk / 8; ++jj) {
                float cf[8];
                codes8<BITS>(wq[a], jj, cf);
#pragma unroll
                for (int tt = 0; tt < MT; ++tt) {
                    if (tt >= nt) break;
                    // two 16-byte broadcasts instead of eight scalar ones: the shared-memory pipe was this kernel's limit
                    const float4 *hv = reinterpret_cast<const float4 *>(hs + tt * r + c * kChunk + jj * 8);
                    const float4 h0 = hv[0], h1 = hv[1];
                    const float hf[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                    for (int k = 0; k < 8; ++k) dsum[tt] = fmaf(hf[k], cf[k], dsum[tt]);
                }
            }
#pragma unroll
            for (int tt = 0; tt < MT; ++tt)
                if (tt < nt) acc[tt] = fmaf(sc[a], dsum[tt], fmaf(mn[a], hsum[tt * chunks + c], acc[tt]));
            if (c + kUpAhead < chunks) fetch(a, c + kUpAhead);  // the slot's codes are spent: the chunk four ahead
        }
    }
    if (j < d) {
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
    SXB_CHECK((w->K / kChunk) % kParts == 0, fn, ": H*d = ", w->K, " must be a multiple of ", kChunk * kParts, " (eight parts of whole chunks a row)");
    // Tokens per CTA: as many as shared memory holds (up to four); rows per CTA: so that the grid is one wave of CTAs.
    const size_t es = act == SXB_ACT_F32 ? 4 : 2, per_token = (size_t)w->K * es + (size_t)(w->K / kChunk) * sizeof(float2);
    const size_t fixed = (size_t)kMaxRowGroup * kParts * 4 * sizeof(float) + 64 * sizeof(float);
    int TT = 4;
    while (TT > 1 && (TT * per_token + fixed > 200 * 1024 || TT > T)) TT >>= 1;
    SXB_CHECK(TT * per_token + fixed <= 200 * 1024, fn, ": H*d = ", w->K, " needs ", per_token, " bytes of shared memory a token");
    const int64_t token_groups = (T + TT - 1) / TT;
    int64_t row_groups = std::max<int64_t>(1, std::min<int64_t>(R, sm_count() / token_groups));
    int RG = (int)std::min<int64_t>(kMaxRowGroup, (R + row_groups - 1) / row_groups);
    row_groups = (R + RG - 1) / RG;
    const size_t smem = TT * per_token + fixed;
    auto st = static_cast<cudaStream_t>(stream);
#define SXB_HC_DOWN(TYPE, TTV)                                                                                                         \
    do {                                                                                                                               \
        auto kern = hc_down_kernel<TYPE, BITS, TTV>;                                                                                   \
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory"); \
        const dim3 grid((unsigned)row_groups, (unsigned)token_groups);                                                                 \
        kern<<<grid, kDownThreads, smem, st>>>(static_cast<const TYPE *>(x), w->q, w->scale, w->minv, R, w->K, w->G, d, (int)r, eps, T, RG, h, \
                                               w_in, inv);                                                                             \
    } while (0)
#define SXB_HC_DOWN_T(TYPE)                     \
    do {                                        \
        if (TT == 4) SXB_HC_DOWN(TYPE, 4);      \
        else if (TT == 2) SXB_HC_DOWN(TYPE, 2); \
        else SXB_HC_DOWN(TYPE, 1);              \
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
