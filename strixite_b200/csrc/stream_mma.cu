// Streaming expert / dense kernels for the HBM-bound regime (decode and small ragged batches; also the exact-product
// path at any size).  C ABI twins of the launchers in kernels/linear_q4.hpp, kernels/linear_q8.hpp and of the
// MoeMath::F32 / WmmaBf16 forms of kernels/moe_grouped.hpp.
//
// What the reference does (kernels/linear_q4.hip:175-199): a wave walks one weight row, every lane takes 32 codes per
// 16-byte load and forms s * sum(x*q) + m * sum(x) per chunk with one FMA per weight, then a wave-shuffle reduction.
// On B200 that form is issue-bound long before HBM is: at 6.5 TB/s an SM receives ~46 codes per clock, and one FMA plus
// the nibble -> float conversion per code and per token already exceeds the 128 FP32 lanes.
//
// This kernel keeps the same arithmetic - exact products of BF16 activations with the integer codes, FP32 sums, scale
// and min applied per group in FP32 - but lets the tensor cores form the products:
//   * a warp owns 16 weight rows; lane (g = lane / 4, c = lane % 4) streams rows g and g + 8 with one 16-byte
//     `ld.global.nc` each per step, the four lanes of a quad covering 64 contiguous bytes of a row, which for the
//     served formats (Q4 G = 128, Q8 G = 64) is exactly one quantization group;
//   * nibbles become BF16 pairs in registers with a shift, a `lop3` and a packed subtract per pair:
//     (w >> 4s) & 0x000F000F | 0x43004300 is the pair (128 + code, 128 + code') exactly, minus (128, 128) the codes;
//     a Q8 byte is split into its two nibbles and the high one meets 16 * x;
//   * the activations of the tile's <= 8 tokens sit in shared memory already permuted into `mma.m16n8k16` B-fragment
//     order, so a lane fetches its fragments with conflict-free 16-byte loads; k is permuted consistently on both
//     operands, which a dot product does not notice;
//   * per step: D = sum over the quad's codes of q * x on the tensor cores (exact products, FP32 sums), then
//     acc += s * D + m * sum(x) in FP32.
// Work is cut into units of 16 rows x one tile of <= 8 tokens of one expert; CTAs take contiguous ranges of units so
// a CTA restages activations only when it crosses into another tile, and every touched expert's weights are read
// once per tile (once in total when an expert has <= 8 tokens, the decode case).

#include "experts.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace sxb {
namespace {

constexpr int kThreads = 256;      // small launches: two CTAs of eight warps an SM
constexpr int kBigThreads = 512;   // launches with work for every SM: one CTA of sixteen warps, units handed out on demand
constexpr int kTileTokens = 8;
constexpr int kPrefetch = 4;  // steps of weights in flight per warp beyond the one being consumed
constexpr int64_t kMaxK = 1 << 24;
constexpr int64_t kMaxN = 0x7fffffff;
constexpr size_t kMaxDynSmem = 200 * 1024;

enum Mode { kGather = 0, kSwiglu = 1, kPartial = 2 };
enum Src { kFromWs = 0, kFromSlots = 1, kDense = 2, kPerToken = 3 };

template <int BITS, int G>
struct Geo {
    static constexpr int kCodesPerLane = (BITS == 4 ? 32 : 16) < G / 4 ? (BITS == 4 ? 32 : 16) : G / 4;
    static constexpr int kLoadBytes = kCodesPerLane * BITS / 8;  // 16, 8 or 4
    static constexpr int kWords = kLoadBytes / 4;
    static constexpr int kStepCodes = 4 * kCodesPerLane;  // codes of one row a quad consumes per step (<= G)
    static constexpr int kUnits = kCodesPerLane / 8;      // 16-byte activation units per lane per step
    static constexpr int kStepsPerGroup = G / kStepCodes;
};

template <int WORDS> __device__ inline void load_codes(uint32_t (&w)[WORDS], const uint8_t *p, bool pred);
template <> __device__ inline void load_codes<4>(uint32_t (&w)[4], const uint8_t *p, bool pred) {
    w[0] = w[1] = w[2] = w[3] = 0u;
    if (pred)
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                     : "l"(p));
}
template <> __device__ inline void load_codes<2>(uint32_t (&w)[2], const uint8_t *p, bool pred) {
    w[0] = w[1] = 0u;
    if (pred) asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "l"(p));
}
template <> __device__ inline void load_codes<1>(uint32_t (&w)[1], const uint8_t *p, bool pred) {
    w[0] = 0u;
    if (pred) asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(w[0]) : "l"(p));
}

// D = A * B (no accumulator input: the zero operand needs no registers set up).
__device__ inline void mma_bf16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ inline void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Nibbles s and s + 4 of w as the BF16 pair (n_s, n_{s+4}): `(w >> 4s) & 0x000F000F | 0x43004300` is the pair
// (128 + n_s, 128 + n_{s+4}) exactly (BF16 keeps 8 significant bits), and one packed subtract removes the 128s.
template <int S> __device__ inline uint32_t nibble_pair(uint32_t w) {
    uint32_t v = ((w >> (4 * S)) & 0x000F000Fu) | 0x43004300u, r;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(0x43004300u));
    return r;
}

// Nibbles s and s + 4 of w as the BF16 pair (16 + n_s, 16 + n_{s+4}): the nibble lands in the top four of the seven
// mantissa bits of 16.0 (0x4180), whose steps are 1/8, so the value is 16 + n exactly - a shift and a lop3, no subtract.
// The 16s are taken out after the contraction: sum((16 + n) x) = sum(n x) + 16 sum(x), and sum(x) of the group is at hand
// for the min term anyway.
template <int S> __device__ inline uint32_t nibble_pair16(uint32_t w) {
    const uint32_t sh = S == 0 ? (w << 3) : (w >> (4 * S - 3));
    return (sh & 0x00780078u) | 0x41804180u;
}

__device__ inline uint32_t times16(uint32_t bf16x2) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162 *>(&bf16x2);
    v = __hmul2(v, __float2bfloat162_rn(16.f));
    return *reinterpret_cast<uint32_t *>(&v);
}

struct StreamArgs {
    const uint16_t *x;  // BF16 activations: x [M, K] (gather / dense) or h [M*A, K] (partial)
    const uint8_t *q;
    const uint16_t *scale, *minv;
    int64_t N, K;        // rows per expert, codes per row
    int64_t M, A, E;     // tokens, slots per token, experts in the view
    const int32_t *ws;   // kFromWs
    RouteWords L;
    const int32_t *ids;  // kFromSlots, kPerToken
    const float *coef;   // kPerToken
    void *out;
    uint32_t *err;
};

template <typename T> __device__ inline void store_out(T *p, int64_t i, float v) { store_from_f32(p, i, v); }

// Stages up to 8 activation rows (rows[n] < 0 = none, zeros) into fragment order at xs / xsum.  All threads of the CTA.
template <int BITS, int G>
__device__ inline void stage_tile(const uint16_t *__restrict__ x, int K, const int64_t *rows, uint4 *xs, float *xsum) {
    using geo = Geo<BITS, G>;
    constexpr int UNITS = geo::kUnits, KI = geo::kStepCodes, CPL = geo::kCodesPerLane;
    const int units_per_row = K / 8, steps = K / KI;
    // 8 consecutive k of token n (16 bytes) -> one unit, permuted to match the nibble pairs of the weights.  Four loads a
    // thread are issued before the first is used (see the note on batches below).
    const int n_units = kTileTokens * units_per_row, stride = (int)blockDim.x;
    for (int base = threadIdx.x; base < n_units; base += 4 * stride) {
        uint4 src[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int idx = base + j * stride;
            src[j] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < n_units) {
                const int64_t row = rows[idx / units_per_row];
                if (row >= 0) src[j] = *reinterpret_cast<const uint4 *>(x + row * K + (idx % units_per_row) * 8);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int idx = base + j * stride;
            if (idx >= n_units) break;
            const int n = idx / units_per_row, k = (idx % units_per_row) * 8;
            const int step = k / KI, rem = k % KI, cc = rem / CPL, v = (rem % CPL) / 8;
            uint4 dst;
            if (BITS == 4) {  // [x0 x4 | x1 x5 | x2 x6 | x3 x7]
                dst.x = __byte_perm(src[j].x, src[j].z, 0x5410), dst.y = __byte_perm(src[j].x, src[j].z, 0x7632);
                dst.z = __byte_perm(src[j].y, src[j].w, 0x5410), dst.w = __byte_perm(src[j].y, src[j].w, 0x7632);
            } else {  // [x0 x2 | x1 x3 | x4 x6 | x5 x7]
                dst.x = __byte_perm(src[j].x, src[j].y, 0x5410), dst.y = __byte_perm(src[j].x, src[j].y, 0x7632);
                dst.z = __byte_perm(src[j].z, src[j].w, 0x5410), dst.w = __byte_perm(src[j].z, src[j].w, 0x7632);
            }
            xs[(step * UNITS + v) * 32 + n * 4 + cc] = dst;
        }
    }
    // sum(x) of every (step, token), in a fixed order.
    for (int idx = threadIdx.x; idx < steps * kTileTokens; idx += blockDim.x) {
        const int step = idx / kTileTokens, n = idx % kTileTokens;
        const int64_t row = rows[n];
        float sum = 0.f;
        if (row >= 0) {
            // the loads of a batch are independent of one another: under a streaming kernel's load an L2 round trip is
            // thousands of cycles, and one load at a time made staging a tenth of a decode kernel's time
            const uint4 *p = reinterpret_cast<const uint4 *>(x + row * K + (int64_t)step * KI);
            constexpr int kBatch = KI / 8 < 8 ? KI / 8 : 8;
            for (int i0 = 0; i0 < KI / 8; i0 += kBatch) {
                uint4 u[kBatch];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) u[i] = p[i0 + i];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const uint32_t w4[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) sum += __uint_as_float(w4[j] << 16), sum += __uint_as_float(w4[j] & 0xffff0000u);
                }
            }
        }
        xsum[idx] = sum;
    }
}

// One warp: the dots of weight rows rowa / rowb (lane quad g streams both) with the staged tokens.
// acc[0], acc[1] = row a x tokens 2c, 2c+1;  acc[2], acc[3] = row b x the same tokens.
// VEC: a step is one quantization group and the row has a multiple of four groups, so the scales and mins of the four
// steps of a prefetch block are one aligned 8-byte load each (four loads a block instead of sixteen 2-byte ones).
template <int BITS, int G, bool VEC>
__device__ inline void rows_dot_impl(float (&acc)[4], const StreamArgs &a, int64_t rowa, int64_t rowb, bool va, bool vb,
                                     const uint4 *xs, const float *xsum, int lane) {
    using geo = Geo<BITS, G>;
    constexpr int W = geo::kWords, UNITS = geo::kUnits, KI = geo::kStepCodes;
    static_assert(kPrefetch == 4, "the vector scale path loads four groups at a time");
    const int K = (int)a.K, steps = K / KI, groups = K / G, c = lane & 3;
    const int64_t row_bytes = BITS == 4 ? a.K / 2 : a.K;
    const uint8_t *pa = a.q + rowa * row_bytes + c * geo::kLoadBytes;
    const uint8_t *pb = a.q + rowb * row_bytes + c * geo::kLoadBytes;
    const uint16_t *sa = a.scale + rowa * groups, *ma = a.minv + rowa * groups;
    const uint16_t *sb = a.scale + rowb * groups, *mb = a.minv + rowb * groups;

    uint32_t wa[kPrefetch][W], wb[kPrefetch][W];
    uint16_t qs[VEC ? 1 : kPrefetch][4];
    uint2 qv[2][4];  // VEC: {scale a, min a, scale b, min b} of the block in use and of the next one
    auto fetch = [&](int slot, int step) {
        const bool in = step < steps;
        load_codes<W>(wa[slot], pa + (int64_t)step * 4 * geo::kLoadBytes, in && va);
        load_codes<W>(wb[slot], pb + (int64_t)step * 4 * geo::kLoadBytes, in && vb);
        if (!VEC) {
            const int grp = step / geo::kStepsPerGroup;
            qs[slot][0] = in && va ? __ldg(sa + grp) : (uint16_t)0;
            qs[slot][1] = in && va ? __ldg(ma + grp) : (uint16_t)0;
            qs[slot][2] = in && vb ? __ldg(sb + grp) : (uint16_t)0;
            qs[slot][3] = in && vb ? __ldg(mb + grp) : (uint16_t)0;
        }
    };
    auto fetch_scales = [&](uint2 (&dst)[4], int step0) {  // VEC: the four groups step0 .. step0 + 3
        const bool in = step0 < steps;
        const uint2 z = make_uint2(0u, 0u);
        dst[0] = in && va ? __ldg(reinterpret_cast<const uint2 *>(sa + step0)) : z;
        dst[1] = in && va ? __ldg(reinterpret_cast<const uint2 *>(ma + step0)) : z;
        dst[2] = in && vb ? __ldg(reinterpret_cast<const uint2 *>(sb + step0)) : z;
        dst[3] = in && vb ? __ldg(reinterpret_cast<const uint2 *>(mb + step0)) : z;
    };
    if (VEC) fetch_scales(qv[0], 0);
#pragma unroll
    for (int p = 0; p < kPrefetch; ++p) fetch(p, p);
    for (int step0 = 0; step0 < steps; step0 += kPrefetch) {
        if (VEC) fetch_scales(qv[1], step0 + kPrefetch);
#pragma unroll
        for (int p = 0; p < kPrefetch; ++p) {
            const int step = step0 + p;
            if (step < steps) {
                float d[4] = {0.f, 0.f, 0.f, 0.f};
                const uint4 *xu = xs + (size_t)step * UNITS * 32 + lane;
#pragma unroll
                for (int v = 0; v < UNITS; ++v) {
                    const uint4 bx = xu[v * 32];
                    if (BITS == 4) {
                        const uint32_t x0 = wa[p][v], x1 = wb[p][v];
                        mma_bf16(d, nibble_pair16<0>(x0), nibble_pair16<0>(x1), nibble_pair16<1>(x0), nibble_pair16<1>(x1), bx.x, bx.y);
                        mma_bf16(d, nibble_pair16<2>(x0), nibble_pair16<2>(x1), nibble_pair16<3>(x0), nibble_pair16<3>(x1), bx.z, bx.w);
                    } else {
                        const uint32_t bw[4] = {bx.x, bx.y, bx.z, bx.w};
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t x0 = wa[p][2 * v + h], x1 = wb[p][2 * v + h];
                            mma_bf16(d, nibble_pair<0>(x0), nibble_pair<0>(x1), nibble_pair<1>(x0), nibble_pair<1>(x1),
                                     bw[2 * h], times16(bw[2 * h]));
                            mma_bf16(d, nibble_pair<2>(x0), nibble_pair<2>(x1), nibble_pair<3>(x0), nibble_pair<3>(x1),
                                     bw[2 * h + 1], times16(bw[2 * h + 1]));
                        }
                    }
                }
                const float2 xs2 = *reinterpret_cast<const float2 *>(xsum + step * kTileTokens + 2 * c);
                uint16_t q4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (VEC) q4[i] = (uint16_t)((p < 2 ? qv[0][i].x : qv[0][i].y) >> (16 * (p & 1)));
                    else q4[i] = qs[p][i];
                }
                const float s_a = bf16_bits_to_f32(q4[0]), s_b = bf16_bits_to_f32(q4[2]);
                float m_a = bf16_bits_to_f32(q4[1]), m_b = bf16_bits_to_f32(q4[3]);
                if (BITS == 4) m_a = fmaf(-16.f, s_a, m_a), m_b = fmaf(-16.f, s_b, m_b);  // the 16s of nibble_pair16
                acc[0] = fmaf(s_a, d[0], fmaf(m_a, xs2.x, acc[0]));
                acc[1] = fmaf(s_a, d[1], fmaf(m_a, xs2.y, acc[1]));
                acc[2] = fmaf(s_b, d[2], fmaf(m_b, xs2.x, acc[2]));
                acc[3] = fmaf(s_b, d[3], fmaf(m_b, xs2.y, acc[3]));
            }
            fetch(p, step + kPrefetch);  // refill the slot just consumed
        }
        if (VEC) {
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[0][i] = qv[1][i];
        }
    }
}

// The common shape, kept lean because the kernel saturates the integer pipe before HBM: a step is one group, the row has
// a whole number of four-step blocks, scales and mins come by aligned 8-byte loads.  No per-load predicates (a row past
// the end of the expert is replaced by a row that exists; its sums are dropped by the caller), pointers advance by
// increments, the last block is peeled so nothing is fetched past the end of a row, and a step's first MMA takes a
// zero accumulator operand instead of cleared registers.
template <int BITS, int G>
__device__ inline void rows_dot_fast(float (&acc)[4], const StreamArgs &a, int64_t rowa, int64_t rowb, const uint4 *xs,
                                     const float *xsum, int lane) {
    using geo = Geo<BITS, G>;
    constexpr int W = geo::kWords, UNITS = geo::kUnits, KI = geo::kStepCodes;
    constexpr int kBlockBytes = kPrefetch * 4 * geo::kLoadBytes;  // bytes of one row consumed per block of four steps
    const int K = (int)a.K, blocks = K / (KI * kPrefetch), groups = K / G, c = lane & 3;
    const int64_t row_bytes = BITS == 4 ? a.K / 2 : a.K;
    const uint8_t *pa = a.q + rowa * row_bytes + c * geo::kLoadBytes;
    const uint8_t *pb = a.q + rowb * row_bytes + c * geo::kLoadBytes;
    const uint2 *sa = reinterpret_cast<const uint2 *>(a.scale + rowa * groups), *ma = reinterpret_cast<const uint2 *>(a.minv + rowa * groups);
    const uint2 *sb = reinterpret_cast<const uint2 *>(a.scale + rowb * groups), *mb = reinterpret_cast<const uint2 *>(a.minv + rowb * groups);
    const uint4 *xu = xs + lane;
    const float *xq = xsum + 2 * c;

    uint32_t wa[kPrefetch][W], wb[kPrefetch][W];
    uint2 qv[4], qn[4];  // {scale a, min a, scale b, min b} of the block in use / of the next one
    auto fetch_codes = [&](int p) {  // step p of the block pa / pb point at
        load_codes<W>(wa[p], pa + p * 4 * geo::kLoadBytes, true);
        load_codes<W>(wb[p], pb + p * 4 * geo::kLoadBytes, true);
    };
    auto fetch_scales = [&](uint2 (&dst)[4]) { dst[0] = __ldg(sa), dst[1] = __ldg(ma), dst[2] = __ldg(sb), dst[3] = __ldg(mb); };
    auto consume = [&](int p) {
        float d[4];
#pragma unroll
        for (int v = 0; v < UNITS; ++v) {
            const uint4 bx = xu[(p * UNITS + v) * 32];
            if (BITS == 4) {
                const uint32_t x0 = wa[p][v], x1 = wb[p][v];
                if (v == 0) mma_bf16_first(d, nibble_pair16<0>(x0), nibble_pair16<0>(x1), nibble_pair16<1>(x0), nibble_pair16<1>(x1), bx.x, bx.y);
                else mma_bf16(d, nibble_pair16<0>(x0), nibble_pair16<0>(x1), nibble_pair16<1>(x0), nibble_pair16<1>(x1), bx.x, bx.y);
                mma_bf16(d, nibble_pair16<2>(x0), nibble_pair16<2>(x1), nibble_pair16<3>(x0), nibble_pair16<3>(x1), bx.z, bx.w);
            } else {
                const uint32_t bw[4] = {bx.x, bx.y, bx.z, bx.w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t x0 = wa[p][2 * v + h], x1 = wb[p][2 * v + h];
                    if (v == 0 && h == 0)
                        mma_bf16_first(d, nibble_pair<0>(x0), nibble_pair<0>(x1), nibble_pair<1>(x0), nibble_pair<1>(x1), bw[0], times16(bw[0]));
                    else
                        mma_bf16(d, nibble_pair<0>(x0), nibble_pair<0>(x1), nibble_pair<1>(x0), nibble_pair<1>(x1), bw[2 * h], times16(bw[2 * h]));
                    mma_bf16(d, nibble_pair<2>(x0), nibble_pair<2>(x1), nibble_pair<3>(x0), nibble_pair<3>(x1), bw[2 * h + 1],
                             times16(bw[2 * h + 1]));
                }
            }
        }
        const float2 xs2 = *reinterpret_cast<const float2 *>(xq + p * kTileTokens);
        // BF16 bits -> FP32: the upper half of the word as it is, the lower half shifted up
        auto f32_of = [&](const uint2 &q) { const uint32_t w = p < 2 ? q.x : q.y; return __uint_as_float((p & 1) ? (w & 0xffff0000u) : (w << 16)); };
        const float s_a = f32_of(qv[0]), s_b = f32_of(qv[2]);
        float m_a = f32_of(qv[1]), m_b = f32_of(qv[3]);
        if (BITS == 4) m_a = fmaf(-16.f, s_a, m_a), m_b = fmaf(-16.f, s_b, m_b);  // the 16s of nibble_pair16
        acc[0] = fmaf(s_a, d[0], fmaf(m_a, xs2.x, acc[0]));
        acc[1] = fmaf(s_a, d[1], fmaf(m_a, xs2.y, acc[1]));
        acc[2] = fmaf(s_b, d[2], fmaf(m_b, xs2.x, acc[2]));
        acc[3] = fmaf(s_b, d[3], fmaf(m_b, xs2.y, acc[3]));
    };

    fetch_scales(qv);
#pragma unroll
    for (int p = 0; p < kPrefetch; ++p) fetch_codes(p);
    for (int b = 1; b < blocks; ++b) {  // consume block b - 1, fetching block b into the registers it frees
        pa += kBlockBytes, pb += kBlockBytes, ++sa, ++ma, ++sb, ++mb;
        fetch_scales(qn);
#pragma unroll
        for (int p = 0; p < kPrefetch; ++p) {
            consume(p);
            fetch_codes(p);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = qn[i];
        xu += kPrefetch * UNITS * 32, xq += kPrefetch * kTileTokens;
    }
#pragma unroll
    for (int p = 0; p < kPrefetch; ++p) consume(p);
}

template <int BITS, int G>
__device__ inline void rows_dot(float (&acc)[4], const StreamArgs &a, int64_t rowa, int64_t rowb, bool va, bool vb,
                                const uint4 *xs, const float *xsum, int lane) {
    using geo = Geo<BITS, G>;
    const int groups = (int)(a.K / G);
    const bool vec = geo::kStepsPerGroup == 1 && groups % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(a.scale) | reinterpret_cast<uintptr_t>(a.minv)) & 7) == 0;
    if (vec && geo::kStepsPerGroup == 1) {
        // rows past the end of the expert: stream a row that exists instead (the caller drops their sums)
        const int64_t any = va ? rowa : vb ? rowb : 0;
        rows_dot_fast<BITS, G>(acc, a, va ? rowa : any, vb ? rowb : any, xs, xsum, lane);
    } else {
        rows_dot_impl<BITS, G, false>(acc, a, rowa, rowb, va, vb, xs, xsum, lane);
    }
}

template <int BITS, int G, int MODE, int SRC, typename TOUT>
__global__ void __launch_bounds__(kBigThreads, 1) stream_kernel(const StreamArgs a) {
    using geo = Geo<BITS, G>;
    const int kWarps = (int)blockDim.x >> 5;
    extern __shared__ __align__(16) unsigned char smem[];
    const int K = (int)a.K, steps = K / geo::kStepCodes;
    const size_t pass_bytes = (size_t)steps * geo::kUnits * 512 + (size_t)steps * kTileTokens * 4;
    __shared__ int64_t s_row[kTileTokens];  // activation row of each token of the tile, -1 = none
    __shared__ int64_t s_out[kTileTokens];  // output row (slot, or token for dense)
    __shared__ int s_bucket, s_cnt;
    __shared__ int s_next;  // the next unit of the CTA's run that no warp has taken yet

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
    const int64_t I = a.N / 2;
    const int64_t units_per_tile = MODE == kSwiglu ? (I + 7) / 8 : (a.N + 15) / 16;
    const int64_t n_tiles = SRC == kFromWs      ? a.ws[0]
                            : SRC == kFromSlots ? a.M * a.A
                            : SRC == kDense     ? (a.M + kTileTokens - 1) / kTileTokens
                                                : a.M;
    const int64_t total = n_tiles * units_per_tile;
    TOUT *out = static_cast<TOUT *>(a.out);
    // How the units are dealt to the CTAs.  Even split: CTA b takes units [total b / n, total (b + 1) / n) - every CTA busy,
    // but a CTA whose range crosses a tile boundary stages activations twice.  Tile-aligned: every tile's units are cut into
    // `cpt` equal runs and a CTA takes whole runs, one staging each.  The aligned cut is taken when it leaves (almost) no CTA
    // idle; inside a run the warps take units on demand either way.
    const int64_t nb = gridDim.x;
    int64_t cpt = max((int64_t)1, nb / max(n_tiles, (int64_t)1));
    const int64_t chunk = ((units_per_tile + cpt - 1) / cpt + kWarps - 1) / kWarps * kWarps;
    cpt = (units_per_tile + chunk - 1) / chunk;
    const int64_t n_chunks = n_tiles * cpt;
    const bool aligned = ((n_chunks + nb - 1) / nb) * chunk * 100 <= ((total + nb - 1) / nb) * 115;
    for (int64_t ci = blockIdx.x; ci < (aligned ? n_chunks : nb); ci += nb) {
    int64_t u_begin, u_end;
    if (aligned) {
        u_begin = (ci / cpt) * units_per_tile + (ci % cpt) * chunk;
        u_end = min((ci / cpt + 1) * units_per_tile, u_begin + chunk);
    } else {
        u_begin = total * ci / nb, u_end = total * (ci + 1) / nb;
    }
    for (int64_t tile = u_begin / units_per_tile; tile * units_per_tile < u_end; ++tile) {
        const int64_t lo = max(u_begin, tile * units_per_tile), hi = min(u_end, (tile + 1) * units_per_tile);

        if (SRC == kPerToken) {
            // Per-slot combine (kernels/linear_q4.hip:281-322): the tile is token `tile`; its A slots' h rows are
            // staged eight to a pass, every slot meets its own expert's rows, and y = sum_a coef * dot in slot order.
            const int64_t m = tile;
            const int passes = (int)((a.A + kTileTokens - 1) / kTileTokens);
            __syncthreads();
            if (threadIdx.x == 0) {
                int bad = -1;
                for (int k = 0; k < a.A && bad < 0; ++k)
                    if (a.ids[m * a.A + k] < 0 || a.ids[m * a.A + k] >= a.E) bad = k;
                if (bad >= 0) raise_error(a.err, (uint32_t)a.ids[m * a.A + bad], (uint32_t)(m * a.A + bad));
                s_cnt = bad < 0;
            }
            __syncthreads();
            const bool valid = s_cnt != 0;
            for (int p = 0; valid && p < passes; ++p) {
                __syncthreads();
                if (threadIdx.x < kTileTokens) {
                    const int k = p * kTileTokens + threadIdx.x;
                    s_row[threadIdx.x] = k < a.A ? m * a.A + k : -1;
                }
                __syncthreads();
                stage_tile<BITS, G>(a.x, K, s_row, reinterpret_cast<uint4 *>(smem + p * pass_bytes),
                                    reinterpret_cast<float *>(smem + p * pass_bytes + (size_t)steps * geo::kUnits * 512));
            }
            __syncthreads();
            for (int64_t unit = lo + warp; unit < hi; unit += kWarps) {
                const int64_t u = unit - tile * units_per_tile;
                const int64_t ra = u * 16 + g, rb = ra + 8;
                const bool va = ra < a.N, vb = rb < a.N;
                float ta = 0.f, tb = 0.f;
                for (int k = 0; valid && k < a.A; ++k) {
                    const int p = k / kTileTokens, col = k % kTileTokens;
                    const int64_t base = (int64_t)a.ids[m * a.A + k] * a.N;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    rows_dot<BITS, G>(acc, a, base + ra, base + rb, va, vb, reinterpret_cast<const uint4 *>(smem + p * pass_bytes),
                                      reinterpret_cast<const float *>(smem + p * pass_bytes + (size_t)steps * geo::kUnits * 512),
                                      lane);
                    if (c == col / 2) {  // the lane of the quad that holds this slot's column
                        const float cf = a.coef[m * a.A + k];
                        ta = fmaf(cf, col & 1 ? acc[1] : acc[0], ta);
                        tb = fmaf(cf, col & 1 ? acc[3] : acc[2], tb);
                    }
                }
                // the four lanes of a quad hold the partial sums of slots {0,1}, {2,3}, {4,5}, {6,7} (mod 8)
                ta += __shfl_xor_sync(0xffffffffu, ta, 1), tb += __shfl_xor_sync(0xffffffffu, tb, 1);
                ta += __shfl_xor_sync(0xffffffffu, ta, 2), tb += __shfl_xor_sync(0xffffffffu, tb, 2);
                if (c == 0) {
                    if (va) store_out(out, m * a.N + ra, valid ? ta : qnan_f32());
                    if (vb) store_out(out, m * a.N + rb, valid ? tb : qnan_f32());
                }
            }
            continue;
        }

        __syncthreads();  // every warp is done with the previous tile's shared memory
        if (threadIdx.x < kTileTokens) {
            const int n = threadIdx.x;
            int64_t row = -1, orow = -1;
            if (SRC == kFromWs) {
                const int bucket = a.ws[a.L.t8_bucket + tile], start = a.ws[a.L.t8_start + tile];
                const int cnt = min(kTileTokens, a.ws[a.L.offsets + bucket + 1] - start);
                if (n == 0) s_bucket = bucket, s_cnt = cnt;
                if (n < cnt) {
                    orow = a.ws[a.L.slots + start + n];
                    row = MODE == kPartial ? orow : orow / a.A;
                }
            } else if (SRC == kFromSlots) {
                if (n == 0) {
                    const int32_t id = a.ids[tile];
                    const bool ok = id >= 0 && id < a.E;
                    if (!ok) raise_error(a.err, (uint32_t)id, (uint32_t)tile);
                    s_bucket = ok ? id : (int)a.E, s_cnt = 1;
                    orow = tile;
                    row = MODE == kPartial ? tile : tile / a.A;
                }
            } else {
                const int64_t m = tile * kTileTokens + n;
                if (n == 0) s_bucket = 0, s_cnt = (int)min((int64_t)kTileTokens, a.M - tile * kTileTokens);
                if (m < a.M) row = orow = m;
            }
            s_row[n] = row, s_out[n] = orow;
        }
        __syncthreads();
        const int bucket = s_bucket, cnt = s_cnt;
        const bool valid = bucket < a.E;  // bucket E: slots with an id outside [0, E) - their outputs become NaN
        uint4 *xs = reinterpret_cast<uint4 *>(smem);
        float *xsum = reinterpret_cast<float *>(smem + (size_t)steps * geo::kUnits * 512);
        if (valid) stage_tile<BITS, G>(a.x, K, s_row, xs, xsum);
        if (threadIdx.x == 0) s_next = 0;
        __syncthreads();

        // Warps take units on demand: two warps of an SM do not stream at the same rate (measured: the units of one of two
        // co-resident CTAs took 2.5 times as long as the other's while both were alive), and a fixed deal leaves the fast ones
        // idle at the end.  A unit's result does not depend on which warp computes it.
        for (;;) {
            int taken = 0;
            if (lane == 0) taken = atomicAdd(&s_next, 1);
            taken = __shfl_sync(0xffffffffu, taken, 0);
            const int64_t unit = lo + taken;
            if (unit >= hi) break;
            const int64_t u = unit - tile * units_per_tile;
            // The two weight rows this lane streams, as rows inside the expert, and where their results go.
            int64_t ra, rb;
            bool va, vb;
            if (MODE == kSwiglu) {
                ra = u * 8 + g, rb = I + u * 8 + g;
                va = vb = u * 8 + g < I;
            } else {
                ra = u * 16 + g, rb = ra + 8;
                va = ra < a.N, vb = rb < a.N;
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (valid) rows_dot<BITS, G>(acc, a, (int64_t)bucket * a.N + ra, (int64_t)bucket * a.N + rb, va, vb, xs, xsum, lane);
            // Epilogue.  Lane (g, c) holds rows ra / rb for tokens 2c and 2c + 1.
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int n = 2 * c + t;
                if (n >= cnt) continue;
                const int64_t orow = s_out[n];
                if (MODE == kSwiglu) {
                    if (!va) continue;
                    // kernels/linear_q4.hip:272-274: g, u as stored, h = stored(stored(silu(g)) * u)
                    const float gg = as_stored_bf16(acc[t]), uu = as_stored_bf16(acc[2 + t]);
                    const float hv = as_stored_bf16(silu_f32(gg)) * uu;
                    store_out(out, orow * I + ra, valid ? hv : qnan_f32());
                } else {
                    if (va) store_out(out, orow * a.N + ra, valid ? acc[t] : qnan_f32());
                    if (vb) store_out(out, orow * a.N + rb, valid ? acc[2 + t] : qnan_f32());
                }
            }
        }
    }
    }
}

// y[m, n] = sum_a fma(coef[m, a], partial[m*A + a, n]) in slot order, one rounding (kernels/moe_grouped.hip:948-984).
// Four columns a thread.  A token with an id outside [0, E_total) gets a NaN row.  Slots of experts outside
// [e_lo, e_lo + E_local) - other ranks' in expert-parallel runs - are skipped.  SH folds the shared expert's gated add:
// y = stored(sum) + sigmoid(gate) * s, the arithmetic of moe_shared_add on the stored y.
// PBF16: the per-slot dots are BF16 bits, N * 2 bytes a slot (kernels/moe_grouped.hip:47-57), read from the same buffer.
template <typename TOUT, typename TS, bool SH, bool PBF16>
__global__ void __launch_bounds__(256)
    combine_reduce_kernel(const float *__restrict__ partial, const int32_t *__restrict__ ids, const float *__restrict__ coef,
                          int64_t M, int64_t A, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t N,
                          TOUT *__restrict__ y, const TS *__restrict__ s, const float *__restrict__ gate_logit,
                          int64_t gate_ld, uint32_t gate_index, uint32_t *err) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= M * N) return;
    const int64_t m = i / N, n = i % N;  // N % 4 == 0: the four columns lie in one row
    bool ok = true;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t k = 0; k < A; ++k) {
        const int32_t id = ids[m * A + k];
        ok = ok && id >= 0 && id < E_total;
        if (id < e_lo || id >= e_lo + E_local) continue;
        const float cf = coef[m * A + k];
        float4 p;
        if constexpr (PBF16) {
            const uint2 b = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(partial) + (m * A + k) * N + n);
            p.x = __uint_as_float(b.x << 16), p.y = __uint_as_float(b.x & 0xffff0000u);
            p.z = __uint_as_float(b.y << 16), p.w = __uint_as_float(b.y & 0xffff0000u);
        } else {
            p = *reinterpret_cast<const float4 *>(partial + (m * A + k) * N + n);
        }
        v[0] = fmaf(cf, p.x, v[0]), v[1] = fmaf(cf, p.y, v[1]), v[2] = fmaf(cf, p.z, v[2]), v[3] = fmaf(cf, p.w, v[3]);
    }
    if (!ok) v[0] = v[1] = v[2] = v[3] = qnan_f32();
    if constexpr (SH) {
        const float gl = gate_logit[m * gate_ld];
        const bool gok = isfinite(gl);
        if (!gok && n == 0) raise_error(err, (uint32_t)m, gate_index);
        const float gt = gok ? 1.f / (1.f + expf(-gl)) : qnan_f32();
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = fmaf(gt, load_as_f32(s, i + j), as_stored<TOUT>(v[j]));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) store_from_f32(y, i + j, v[j]);
}

// The same reduce for an expert-parallel rank whose rows go to their owners: no shared add, FP32 sums; the four columns
// are stored, as this rank's piece, into the owner's receive buffer through its peer mapping (16 or 8 bytes a store).
template <bool PBF16, bool OUT_F16>
__global__ void __launch_bounds__(256)
    combine_reduce_peer_kernel(const float *__restrict__ partial, const int32_t *__restrict__ ids, const float *__restrict__ coef,
                               int64_t M, int64_t A, int64_t E_total, int64_t e_lo, int64_t E_local, int64_t N, const PeerOut peer) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= M * N) return;
    const int64_t m = i / N, n = i % N;
    bool ok = true;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t k = 0; k < A; ++k) {
        const int32_t id = ids[m * A + k];
        ok = ok && id >= 0 && id < E_total;
        if (id < e_lo || id >= e_lo + E_local) continue;
        const float cf = coef[m * A + k];
        float4 p;
        if constexpr (PBF16) {
            const uint2 b = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(partial) + (m * A + k) * N + n);
            p.x = __uint_as_float(b.x << 16), p.y = __uint_as_float(b.x & 0xffff0000u);
            p.z = __uint_as_float(b.y << 16), p.w = __uint_as_float(b.y & 0xffff0000u);
        } else {
            p = *reinterpret_cast<const float4 *>(partial + (m * A + k) * N + n);
        }
        v[0] = fmaf(cf, p.x, v[0]), v[1] = fmaf(cf, p.y, v[1]), v[2] = fmaf(cf, p.z, v[2]), v[3] = fmaf(cf, p.w, v[3]);
    }
    if (!ok) v[0] = v[1] = v[2] = v[3] = qnan_f32();
    const int owner = (int)(m / peer.t);
    const int64_t at = (((int64_t)peer.rank * peer.t + m % peer.t) * N + n);
    if constexpr (OUT_F16) {
        // F16, not BF16: eleven significant bits keep the sum of a row's pieces inside the layer's tolerance (BF16 pieces
        // measured 3.4e-2 of the RMS); a piece beyond F16's range (|v| > 65504) would become infinite
        const __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t *>(&lo), o.y = *reinterpret_cast<const uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(peer.base[owner]) + at) = o;
    } else {
        *reinterpret_cast<float4 *>(static_cast<float *>(peer.base[owner]) + at) = make_float4(v[0], v[1], v[2], v[3]);
    }
    // no fence here: the stores have been performed when the kernel has completed, and the rank signals its peers only by
    // work enqueued behind this kernel on the same stream
}

int check_view(const char *fn, const SxbQView *w) {
    SXB_CHECK(w != nullptr, fn, ": null weight view");
    SXB_CHECK(w->q != nullptr && w->scale != nullptr && w->minv != nullptr, fn, ": null weight pointer (q=",
              (const void *)w->q, ", scale=", (const void *)w->scale, ", min=", (const void *)w->minv, ")");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->N >= 1 && w->N <= kMaxN, fn, ": N = ", w->N, ", expected 1..", kMaxN);
    SXB_CHECK(w->K >= w->G && w->K <= kMaxK && w->K % w->G == 0, fn, ": K = ", w->K,
              " must be a positive multiple of group size ", w->G, " and <= ", kMaxK);
    SXB_CHECK(aligned16(w->q), fn, ": code array ", (const void *)w->q, " must be 16-byte aligned for vector loads");
    SXB_CHECK(reinterpret_cast<uintptr_t>(w->scale) % 2 == 0 && reinterpret_cast<uintptr_t>(w->minv) % 2 == 0, fn,
              ": scale / min arrays must be 2-byte aligned");
    return SXB_OK;
}

template <int BITS, int G, int MODE, int SRC, typename TOUT>
int launch_stream(const char *fn, const StreamArgs &a, int64_t est_units, cudaStream_t st) {
    using geo = Geo<BITS, G>;
    const int64_t steps = a.K / geo::kStepCodes;
    const int64_t passes = SRC == kPerToken ? (a.A + kTileTokens - 1) / kTileTokens : 1;
    const size_t smem = (size_t)passes * ((size_t)steps * geo::kUnits * 512 + (size_t)steps * kTileTokens * 4);
    SXB_CHECK(smem <= kMaxDynSmem, fn, ": K = ", a.K, SRC == kPerToken ? " x A = " : "", SRC == kPerToken ? a.A : 0, " needs ", smem,
              " bytes of shared memory for one tile's activations, more than ", kMaxDynSmem,
              " (K * 16 * ceil(A / 8) bytes for the per-slot combine, K * 16 otherwise; use the grouped form)");
    auto kern = stream_kernel<BITS, G, MODE, SRC, TOUT>;
    SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn,
             ": reserving shared memory");
    // One CTA of sixteen warps an SM when there are several units for every warp of the machine; otherwise CTAs of eight
    // warps, two an SM where their shared memory allows, and never more CTAs than one per unit and warp.
    const bool big = est_units >= (int64_t)sm_count() * (kBigThreads / 32) * 2;
    const int threads = big ? kBigThreads : kThreads, warps = threads / 32;
    const int per_sm = big || smem > 100 * 1024 ? 1 : 2;
    int64_t grid = (int64_t)sm_count() * per_sm;
    grid = std::max<int64_t>(1, std::min<int64_t>(grid, (est_units + warps - 1) / warps));
    kern<<<(unsigned)grid, threads, smem, st>>>(a);
    return SXB_OK;
}

template <int BITS, int MODE, int SRC, typename TOUT>
int launch_by_group(const char *fn, const StreamArgs &a, int64_t G, int64_t est_units, cudaStream_t st) {
    switch (G) {
        case 32: return launch_stream<BITS, 32, MODE, SRC, TOUT>(fn, a, est_units, st);
        case 64: return launch_stream<BITS, 64, MODE, SRC, TOUT>(fn, a, est_units, st);
        default: return launch_stream<BITS, 128, MODE, SRC, TOUT>(fn, a, est_units, st);
    }
}

int need_bf16(const char *fn, int act) {
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SXB_CHECK(act == SXB_ACT_BF16, fn,
              ": FP32 activations are not implemented by the sm_100a expert kernels (BF16 activations only)");
    return SXB_OK;
}

// Dense y = x W^T.
template <int BITS>
int linear_impl(const char *fn, const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act,
                sxb_stream_t stream) {
    SXB_CHECK(x != nullptr && y != nullptr, fn, ": null pointer (x=", x, ", y=", y, ")");
    if (int rc = check_view(fn, w)) return rc;
    SXB_CHECK(M >= 1 && M <= 65535ll * 8, fn, ": M (rows of x) = ", M, ", expected 1..", 65535ll * 8);
    SXB_CHECK(aligned16(x), fn, ": x ", x, " must be 16-byte aligned for vector loads");
    SXB_CHECK(act_ok(act) && (out_act == act || out_act == SXB_ACT_F32), fn, ": output dtype ", act_name(out_act), " with input ",
              act_name(act), " unsupported (same dtype, or BF16 -> F32)");
    if (act == SXB_ACT_F32) {
        SXB_CHECK(apart(x, M * w->K * 4, y, M * w->N * 4), fn, ": output y overlaps input x");
        return f32_gather<BITS>(fn, x, w, 1, nullptr, nullptr, M, 1, y, false, 1, nullptr, stream);
    }
    if (int rc = need_bf16(fn, act)) return rc;
    SXB_CHECK(apart(x, M * w->K * 2, y, M * w->N * act_bytes(out_act)), fn, ": output y [", y, ", +",
              M * w->N * act_bytes(out_act), " B) overlaps input x [", x, ", +", M * w->K * 2, " B)");
    StreamArgs a{};
    a.x = static_cast<const uint16_t *>(x), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = w->N, a.K = w->K, a.M = M, a.A = 1, a.E = 1, a.out = y;
    const int64_t units = ((M + 7) / 8) * ((w->N + 15) / 16);
    auto st = static_cast<cudaStream_t>(stream);
    int rc = out_act == SXB_ACT_F32 ? launch_by_group<BITS, kGather, kDense, float>(fn, a, w->G, units, st)
                                    : launch_by_group<BITS, kGather, kDense, uint16_t>(fn, a, w->G, units, st);
    if (rc) return rc;
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), "->", act_name(out_act), " M=", M, " N=", w->N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

int check_experts(const char *fn, const void *x, const SxbQView *w, int64_t E, int64_t M, int64_t A, const void *y) {
    SXB_CHECK(x != nullptr && y != nullptr, fn, ": null pointer (x=", x, ", y=", y, ")");
    if (int rc = check_view(fn, w)) return rc;
    SXB_CHECK(E >= 1 && w->N % E == 0, fn, ": weight has ", w->N, " rows, not a multiple of E = ", E, " experts");
    SXB_CHECK(A >= 1 && A <= 64 && A <= E, fn, ": A (active experts per token) = ", A, ", expected 1..min(64, E=", E, ")");
    SXB_CHECK(aligned16(x), fn, ": input ", x, " must be 16-byte aligned");
    return SXB_OK;
}

// Per-slot gather (optionally with SwiGLU): kernels/linear_q4.hip:420-453.
template <int BITS>
int experts_slots_impl(const char *fn, const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M,
                       int64_t A, void *y, int act, uint32_t *err, sxb_stream_t stream, bool swiglu) {
    if (int rc = check_experts(fn, x, w, E, M, A, y)) return rc;
    SXB_CHECK(ids != nullptr && err != nullptr, fn, ": null pointer (ids=", (const void *)ids, ", err=", (const void *)err, ")");
    SXB_CHECK(M >= 1 && M <= 65535, fn, ": M (tokens) = ", M, ", expected 1..65535");
    if (act == SXB_ACT_F32) {
        SXB_CHECK(apart(x, M * w->K * 4, y, M * A * (swiglu ? w->N / E / 2 : w->N / E) * 4), fn, ": output overlaps input");
        return f32_gather<BITS>(fn, x, w, E, ids, nullptr, M, A, y, swiglu, (int)A, err, stream);
    }
    if (int rc = need_bf16(fn, act)) return rc;
    const int64_t N = w->N / E;
    SXB_CHECK(!swiglu || N % 2 == 0, fn, ": SwiGLU gather needs an even row count per expert ([gate | up]), got ", N);
    SXB_CHECK(apart(x, M * w->K * 2, y, M * A * (swiglu ? N / 2 : N) * 2), fn, ": output overlaps input");
    StreamArgs a{};
    a.x = static_cast<const uint16_t *>(x), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = N, a.K = w->K, a.M = M, a.A = A, a.E = E, a.ids = ids, a.out = y, a.err = err;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t units = M * A * (swiglu ? (N / 2 + 7) / 8 : (N + 15) / 16);
    int rc = swiglu ? launch_by_group<BITS, kSwiglu, kFromSlots, uint16_t>(fn, a, w->G, units, st)
                    : launch_by_group<BITS, kGather, kFromSlots, uint16_t>(fn, a, w->G, units, st);
    if (rc) return rc;
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), " M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G,
                     swiglu ? " swiglu" : "");
    return SXB_OK;
}

int check_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, int64_t M, int64_t A, const void *ws,
                  size_t ws_bytes, const void *y) {
    if (int rc = check_experts(fn, x, w, E, M, A, y)) return rc;
    SXB_CHECK(ws != nullptr, fn, ": null workspace");
    SXB_CHECK(E <= kMoeMaxExperts && M * A <= kMoeMaxSlots, fn, ": M = ", M, " tokens x A = ", A, " slots over E = ", E,
              " experts (E <= ", kMoeMaxExperts, ", M*A <= ", kMoeMaxSlots, ")");
    SXB_CHECK(ws_bytes >= (size_t)route_words(M, A, E).total * 4, fn, ": workspace of ", ws_bytes, " bytes, needs ",
              route_words(M, A, E).total * 4, " for M = ", M, ", A = ", A, ", E = ", E);
    return SXB_OK;
}

}  // namespace

// The exact-product grouped forms (MoeMath::F32 / WmmaBf16), shared with grouped.cu's dispatch.
template <int BITS>
int stream_gather_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                          int64_t M, int64_t A, void *y, int act, bool swiglu, sxb_stream_t stream) {
    if (int rc = check_grouped(fn, x, w, E, M, A, ws, ws_bytes, y)) return rc;
    if (act == SXB_ACT_F32) {
        SXB_CHECK(apart(x, M * w->K * 4, y, M * A * (swiglu ? w->N / E / 2 : w->N / E) * 4), fn, ": output overlaps input x");
        return f32_gather<BITS>(fn, x, w, E, nullptr, ws, M, A, y, swiglu, (int)A, nullptr, stream);
    }
    if (int rc = need_bf16(fn, act)) return rc;
    const int64_t N = w->N / E;
    SXB_CHECK(!swiglu || N % 2 == 0, fn, ": gate_up has ", N, " rows an expert, expected an even count (gate rows then up rows)");
    SXB_CHECK(apart(x, M * w->K * 2, y, M * A * (swiglu ? N / 2 : N) * 2), fn, ": output overlaps input x");
    StreamArgs a{};
    a.x = static_cast<const uint16_t *>(x), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = N, a.K = w->K, a.M = M, a.A = A, a.E = E, a.ws = static_cast<const int32_t *>(ws), a.L = route_words(M, A, E);
    a.out = y;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t units = (M * A / 8 + std::min<int64_t>(E, M * A)) * (swiglu ? (N / 2 + 7) / 8 : (N + 15) / 16);
    int rc = swiglu ? launch_by_group<BITS, kSwiglu, kFromWs, uint16_t>(fn, a, w->G, units, st)
                    : launch_by_group<BITS, kGather, kFromWs, uint16_t>(fn, a, w->G, units, st);
    if (rc) return rc;
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), " M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

template <int BITS>
int stream_partial_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes,
                           int64_t M, int64_t A, float *partial, int act, sxb_stream_t stream) {
    if (int rc = check_grouped(fn, h, w, E, M, A, ws, ws_bytes, partial)) return rc;
    if (act == SXB_ACT_F32) return f32_gather<BITS>(fn, h, w, E, nullptr, ws, M, A, partial, false, 1, nullptr, stream);
    if (int rc = need_bf16(fn, act)) return rc;
    const int64_t N = w->N / E;
    StreamArgs a{};
    a.x = static_cast<const uint16_t *>(h), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = N, a.K = w->K, a.M = M, a.A = A, a.E = E, a.ws = static_cast<const int32_t *>(ws), a.L = route_words(M, A, E);
    a.out = partial;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t units = (M * A / 8 + std::min<int64_t>(E, M * A)) * ((N + 15) / 16);
    if (int rc = launch_by_group<BITS, kPartial, kFromWs, float>(fn, a, w->G, units, st)) return rc;
    SXB_CHECK_LAUNCH(fn, " partial M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

// Per-slot combine without scratch (kernels/linear_q4.hpp:44-46).
template <int BITS>
int stream_combine_slots(const char *fn, const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                         const float *coef, int64_t M, int64_t A, void *y, int act, int out_act, uint32_t *err,
                         sxb_stream_t stream) {
    SXB_CHECK(coef != nullptr, fn, ": null coef");
    if (int rc = check_experts(fn, h, w, E, M, A, y)) return rc;
    SXB_CHECK(ids != nullptr && err != nullptr, fn, ": null pointer (ids=", (const void *)ids, ", err=", (const void *)err, ")");
    SXB_CHECK(M >= 1 && M <= 65535, fn, ": M (tokens) = ", M, ", expected 1..65535");
    SXB_CHECK(act_ok(act) && (out_act == act || out_act == SXB_ACT_F32), fn, ": output dtype ", act_name(out_act), " with activations ",
              act_name(act), " unsupported (same dtype, or F32)");
    if (act == SXB_ACT_F32) {
        SXB_CHECK(apart(h, M * A * w->K * 4, y, M * (w->N / E) * 4), fn, ": output y overlaps input h");
        return f32_combine<BITS>(fn, h, w, E, ids, coef, M, A, y, err, stream);
    }
    if (int rc = need_bf16(fn, act)) return rc;
    const int64_t N = w->N / E;
    SXB_CHECK(apart(h, M * A * w->K * 2, y, M * N * act_bytes(out_act)), fn, ": output y overlaps input h");
    StreamArgs a{};
    a.x = static_cast<const uint16_t *>(h), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = N, a.K = w->K, a.M = M, a.A = A, a.E = E, a.ids = ids, a.coef = coef, a.out = y, a.err = err;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t units = M * ((N + 15) / 16);
    int rc = out_act == SXB_ACT_F32 ? launch_by_group<BITS, kGather, kPerToken, float>(fn, a, w->G, units, st)
                                    : launch_by_group<BITS, kGather, kPerToken, uint16_t>(fn, a, w->G, units, st);
    if (rc) return rc;
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), " M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

template int stream_combine_slots<4>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const float *,
                                     int64_t, int64_t, void *, int, int, uint32_t *, sxb_stream_t);
template int stream_combine_slots<8>(const char *, const void *, const SxbQView *, int64_t, const int32_t *, const float *,
                                     int64_t, int64_t, void *, int, int, uint32_t *, sxb_stream_t);

template int stream_gather_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t,
                                      int64_t, void *, int, bool, sxb_stream_t);
template int stream_gather_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t,
                                      int64_t, void *, int, bool, sxb_stream_t);
template int stream_partial_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t,
                                       int64_t, float *, int, sxb_stream_t);
template int stream_partial_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t,
                                       int64_t, float *, int, sxb_stream_t);

int combine_reduce(const char *fn, const float *partial, const int32_t *ids, const float *coef, int64_t M, int64_t A,
                   int64_t E_total, int64_t e_lo, int64_t E_local, int64_t N, void *y, int out_act,
                   const SxbMoeSharedAdd *shared, int s_act, bool partial_bf16, sxb_stream_t stream, const PeerOut *peer) {
    if (peer != nullptr) {
        SXB_CHECK(partial != nullptr && ids != nullptr && coef != nullptr, fn, ": null pointer");
        SXB_CHECK(shared == nullptr && N % 4 == 0 && aligned16(partial), fn, ": peer output takes no shared add; N = ", N);
        SXB_CHECK(peer->world >= 1 && peer->world <= 8 && peer->t >= 1 && M == peer->t * peer->world, fn, ": ", M, " rows over ",
                  peer->world, " ranks of ", peer->t);
        const unsigned blocks = (unsigned)((M * N / 4 + 255) / 256);
        auto st = static_cast<cudaStream_t>(stream);
#define SXB_PEER(PB, OB) combine_reduce_peer_kernel<PB, OB><<<blocks, 256, 0, st>>>(partial, ids, coef, M, A, E_total, e_lo, E_local, N, *peer)
        if (partial_bf16) {
            if (peer->f16) SXB_PEER(true, true);
            else SXB_PEER(true, false);
        } else {
            if (peer->f16) SXB_PEER(false, true);
            else SXB_PEER(false, false);
        }
#undef SXB_PEER
        SXB_CHECK_LAUNCH(fn, " reduce to peers M=", M, " A=", A, " N=", N);
        return SXB_OK;
    }
    SXB_CHECK(partial != nullptr && ids != nullptr && coef != nullptr && y != nullptr, fn, ": null pointer (partial=",
              (const void *)partial, ", ids=", (const void *)ids, ", coef=", (const void *)coef, ", y=", y, ")");
    SXB_CHECK(N % 4 == 0 && aligned16(partial), fn, ": N = ", N, " must be a multiple of 4 and partial 16-byte aligned");
    SXB_CHECK(act_ok(out_act), fn, ": unsupported output dtype ", out_act);
    if (shared != nullptr) {
        SXB_CHECK(shared->s != nullptr && shared->gate_logit != nullptr && shared->err != nullptr, fn,
                  ": shared add with a null pointer (s=", shared->s, ", gate_logit=", (const void *)shared->gate_logit,
                  ", err=", (const void *)shared->err, ")");
        SXB_CHECK(shared->gate_ld >= 1, fn, ": shared add gate_ld = ", shared->gate_ld, ", expected >= 1");
        SXB_CHECK(apart(y, M * N * act_bytes(out_act), shared->s, M * N * act_bytes(s_act)), fn, ": y overlaps shared s");
    }
    SXB_CHECK(apart(y, M * N * act_bytes(out_act), partial, M * A * N * 4), fn, ": y overlaps partial");
    const unsigned blocks = (unsigned)((M * N / 4 + 255) / 256);
    auto st = static_cast<cudaStream_t>(stream);
    const float *gl = shared ? shared->gate_logit : nullptr;
    const int64_t gld = shared ? shared->gate_ld : 0;
    const uint32_t gi = shared ? shared->gate_index : 0;
    uint32_t *err = shared ? shared->err : nullptr;
#define SXB_REDUCE_P(TOUT, TS, SH, PB)                                                                                  \
    combine_reduce_kernel<TOUT, TS, SH, PB><<<blocks, 256, 0, st>>>(partial, ids, coef, M, A, E_total, e_lo, E_local, N, \
                                                                    static_cast<TOUT *>(y),                              \
                                                                    static_cast<const TS *>(shared ? shared->s : nullptr), \
                                                                    gl, gld, gi, err)
#define SXB_REDUCE(TOUT, TS, SH)                          \
    do {                                                  \
        if (partial_bf16) SXB_REDUCE_P(TOUT, TS, SH, true); \
        else SXB_REDUCE_P(TOUT, TS, SH, false);            \
    } while (0)
    if (out_act == SXB_ACT_F32) {
        if (!shared) SXB_REDUCE(float, float, false);
        else if (s_act == SXB_ACT_F32) SXB_REDUCE(float, float, true);
        else SXB_REDUCE(float, uint16_t, true);
    } else {
        if (!shared) SXB_REDUCE(uint16_t, uint16_t, false);
        else if (s_act == SXB_ACT_F32) SXB_REDUCE(uint16_t, float, true);
        else SXB_REDUCE(uint16_t, uint16_t, true);
    }
#undef SXB_REDUCE
#undef SXB_REDUCE_P
    SXB_CHECK_LAUNCH(fn, " reduce M=", M, " A=", A, " N=", N, shared ? " +shared" : "");
    return SXB_OK;
}

}  // namespace sxb

using namespace sxb;

extern "C" {

int sxb_linear_q4(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream) {
    return linear_impl<4>("linear_q4", x, w, y, M, act, out_act, stream);
}
int sxb_linear_q8(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream) {
    return linear_impl<8>("linear_q8", x, w, y, M, act, out_act, stream);
}

int sxb_linear_q4_experts_gather(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M, int64_t A,
                                 void *y, int act, uint32_t *err, sxb_stream_t stream) {
    return experts_slots_impl<4>("linear_q4_experts_gather", x, w, E, ids, M, A, y, act, err, stream, false);
}
int sxb_linear_q4_experts_gather_swiglu(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M,
                                        int64_t A, void *h, int act, uint32_t *err, sxb_stream_t stream) {
    return experts_slots_impl<4>("linear_q4_experts_gather_swiglu", x, w, E, ids, M, A, h, act, err, stream, true);
}
int sxb_linear_q8_experts_gather(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M, int64_t A,
                                 void *y, int act, uint32_t *err, sxb_stream_t stream) {
    return experts_slots_impl<8>("linear_q8_experts_gather", x, w, E, ids, M, A, y, act, err, stream, false);
}
int sxb_linear_q8_experts_gather_swiglu(const void *x, const SxbQView *w, int64_t E, const int32_t *ids, int64_t M,
                                        int64_t A, void *h, int act, uint32_t *err, sxb_stream_t stream) {
    return experts_slots_impl<8>("linear_q8_experts_gather_swiglu", x, w, E, ids, M, A, h, act, err, stream, true);
}

}  // extern "C"
