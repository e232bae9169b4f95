// Shared by the two tcgen05 expert kernels (grouped_tc.cu: activations gathered per tile, any layout; grouped_tc_tiled.cu:
// tile-blocked activations, one dequantization of the weights shared by up to 256 tokens): launch arguments, output modes,
// and the dequantization of packed codes to the F16 operand.
#pragma once

#include "experts.cuh"
#include "tc_ptx.cuh"

namespace sxb {

// kTcPartialBf16: kTcPartial with the per-slot dots stored as BF16 bits (N * 2 bytes a slot) - for the epilogue it is the
// plain gather's store on h rows.  A mode of its own, so that the per-token store code of every mode stays one short form.
// kTcHcUp: a dense projection whose epilogue is the stream combine of the hyper-connection up mix (TcHcUp below); the
// kernel for tile-blocked activations only.
enum TcMode { kTcGather = 0, kTcSwiglu = 1, kTcPartial = 2, kTcPartialBf16 = 3, kTcHcUp = 4 };

// kTcHcUp (kernels/hc_wmma.hip:244-272): the weight's rows are W_up's rows in the order that puts the H = 4 streams of an
// output column into adjacent tensor-memory lanes - row rb * 128 + q * 32 + l is stream l & 3 of column
// rb * 32 + q * 8 + (l >> 2) - so that a lane finishes z -> sigmoid(z) * x * inv * (1 + norm_w) for its stream and two
// shuffles add the four streams: u[t, j] = (1/4) sum_s ..., rounded once to the activation dtype.  No z in memory.
struct TcHcUp {
    const void *x;        // the streams X [M, 4 d], FP32 or BF16
    const float *inv;     // [M, 4]
    const float *norm_w;  // [4 d]
    void *u;              // [M, d] in x's dtype
    int64_t d;
    int f32;              // x and u are FP32 (else BF16)
};

struct TcArgs {
    const uint16_t *x;  // activations: BF16 or F16 bits, see x_kind
    const uint8_t *q;
    const uint16_t *scale, *minv;
    int64_t N, K;     // weight rows per expert, codes per row
    int64_t A, E;     // slots per token, experts in the view
    const int32_t *ws;
    RouteWords L;
    void *out;
    int x_kind;   // activations: 0 BF16, 1 F16 in natural k order, 2 F16 in this weight operand's k order (staged),
                  // 3 F16 "tile-blocked" (see tiled_offset): one bulk copy per k-block
    int out_f16;  // SwiGLU output h: 0 BF16, 1 F16 bits of its BF16 rounding, 2 the same in the Q4 operand's k order,
                  // 3 / 4 tile-blocked for a Q4 / Q8 down operand
    uint32_t *status;  // >= 3 words: {2, item, role} on a wait that ran out
    int64_t dense_M;   // > 0: a dense projection - no grouping workspace, one group holding rows 0 .. dense_M - 1 in order
    unsigned long long wait_limit_ns;  // bound of every device-side wait
    int test_skip_slot;  // >= 0: CTA 0 never issues ring slot number test_skip_slot, so a wait runs out (tests only)
    TcHcUp hc;           // kTcHcUp only
};

// Eight weights = one 16-byte chunk of the A line, from one word of Q4 codes or two words of Q8 codes.
// w = code * s + m with one F16 rounding (kernels/wmma_gemm.hpp:116-129).
__device__ inline uint4 dequant_q4_word(uint32_t w, __half2 s, __half2 s16, __half2 m) {
    const __half2 k1024 = __float2half2_rn(1024.f);
    const uint32_t w8 = w >> 8;
    // (w & 0x000F000F) | 0x64006400 = (1024 + n0, 1024 + n4); the 0x00F0 nibbles give 1024 + 16 n and meet s / 16
    const __half2 p0 = __hsub2(u32_as_h2((w & 0x000F000Fu) | 0x64006400u), k1024);
    const __half2 p1 = __hsub2(u32_as_h2((w & 0x00F000F0u) | 0x64006400u), k1024);
    const __half2 p2 = __hsub2(u32_as_h2((w8 & 0x000F000Fu) | 0x64006400u), k1024);
    const __half2 p3 = __hsub2(u32_as_h2((w8 & 0x00F000F0u) | 0x64006400u), k1024);
    uint4 d;
    d.x = h2_as_u32(__hfma2(p0, s, m)), d.y = h2_as_u32(__hfma2(p1, s16, m));
    d.z = h2_as_u32(__hfma2(p2, s, m)), d.w = h2_as_u32(__hfma2(p3, s16, m));
    return d;
}
__device__ inline uint4 dequant_q8_words(uint32_t w0, uint32_t w1, __half2 s, __half2 m) {
    const __half2 k1024 = __float2half2_rn(1024.f);
    uint4 d;  // __byte_perm(w, 0x64646464, 0x4140) = (0x6400 | b0, 0x6400 | b1) = (1024 + b0, 1024 + b1)
    d.x = h2_as_u32(__hfma2(__hsub2(u32_as_h2(__byte_perm(w0, 0x64646464u, 0x4140)), k1024), s, m));
    d.y = h2_as_u32(__hfma2(__hsub2(u32_as_h2(__byte_perm(w0, 0x64646464u, 0x4342)), k1024), s, m));
    d.z = h2_as_u32(__hfma2(__hsub2(u32_as_h2(__byte_perm(w1, 0x64646464u, 0x4140)), k1024), s, m));
    d.w = h2_as_u32(__hfma2(__hsub2(u32_as_h2(__byte_perm(w1, 0x64646464u, 0x4342)), k1024), s, m));
    return d;
}

// grouped_tc_tiled.cu: the kernel for tile-blocked activations (a.x_kind == 3).  Same arguments, same outputs.
template <int BITS, int MODE>
int launch_tiled_tc(const char *fn, TcArgs a, int64_t G, cudaStream_t st);

}  // namespace sxb
