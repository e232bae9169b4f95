// Q4 / Q8 quantizers for weights resident on the device; twins of quantize_q4 (formats/q4.cpp:44-88) and quantize_q8
// (formats/q8.cpp:43-82) with bit-identical output: per group of G weights along K, s = bf16((max - min) / levels),
// m = bf16(min), code = clamp(round_half_even((w - m) / s), 0, levels), a constant group (s == 0) gets code 0.  IEEE
// division and rint keep every intermediate equal to the host's.
//
// One warp per group: G / 32 weights a lane, min / max by warp reduction, and each lane packs its own codes, so the
// stores are 32-bit (Q8, G = 128), 16-bit or 8-bit and a group's bytes are written as one contiguous run.

#include "common.cuh"

namespace sxb {
namespace {

constexpr int kThreads = 256;

template <int BITS, int G>
__global__ void __launch_bounds__(kThreads)
    quantize_kernel(const float *__restrict__ w, int64_t n_groups, int64_t groups_per_row, uint8_t *__restrict__ q,
                    uint16_t *__restrict__ scale, uint16_t *__restrict__ minv, uint32_t *err) {
    constexpr int PER = G / 32;  // consecutive weights a lane owns: 1, 2 or 4
    constexpr float kLevels = BITS == 4 ? 15.f : 255.f;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5, n_warps = ((int64_t)gridDim.x * kThreads) >> 5;
    for (int64_t grp = warp0; grp < n_groups; grp += n_warps) {
        const float *src = w + grp * G + lane * PER;
        float v[PER];
        float lo, hi;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            v[i] = src[i];
            bad = bad || !isfinite(v[i]);
        }
        lo = hi = v[0];
#pragma unroll
        for (int i = 1; i < PER; ++i) lo = fminf(lo, v[i]), hi = fmaxf(hi, v[i]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
        }
        if (__any_sync(0xffffffffu, bad)) {
            if (bad) raise_error(err, (uint32_t)(grp / groups_per_row), (uint32_t)((grp % groups_per_row) * G + lane * PER));
        }
        const uint16_t s_bits = f32_to_bf16_bits(__fdiv_rn(__fsub_rn(hi, lo), kLevels)), m_bits = f32_to_bf16_bits(lo);
        const float s = bf16_bits_to_f32(s_bits), m = bf16_bits_to_f32(m_bits);
        if (lane == 0) scale[grp] = s_bits, minv[grp] = m_bits;
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            uint32_t code = 0;
            if (s > 0.f) code = (uint32_t)fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v[i], m), s)), 0.f), kLevels);
            packed |= code << (BITS * i);
        }
        // group grp's codes start at byte grp * G * BITS / 8; the lane's PER codes are PER * BITS bits
        constexpr int kLaneBits = PER * BITS;
        uint8_t *dst = q + grp * (G * BITS / 8);
        if constexpr (kLaneBits == 32) reinterpret_cast<uint32_t *>(dst)[lane] = packed;
        else if constexpr (kLaneBits == 16) reinterpret_cast<uint16_t *>(dst)[lane] = (uint16_t)packed;
        else if constexpr (kLaneBits == 8) dst[lane] = (uint8_t)packed;
        else {  // Q4, G = 32: a nibble a lane - pair neighbouring lanes into a byte
            const uint32_t other = __shfl_down_sync(0xffffffffu, packed, 1);
            if ((lane & 1) == 0) dst[lane >> 1] = (uint8_t)(packed | (other << 4));
        }
    }
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" int sxb_quantize(const float *w, int64_t N, int64_t K, int64_t G, int bits, uint8_t *q, uint16_t *scale,
                            uint16_t *minv, uint32_t *err, sxb_stream_t stream) {
    SXB_CHECK(w != nullptr && q != nullptr && scale != nullptr && minv != nullptr && err != nullptr,
              "quantize: null pointer (w=", (const void *)w, ", q=", (const void *)q, ", scale=", (const void *)scale,
              ", min=", (const void *)minv, ", err=", (const void *)err, ")");
    SXB_CHECK(N >= 1 && K >= 1, "quantize: shape [", N, ", ", K, "] must be positive");
    SXB_CHECK(bits == 4 || bits == 8, "quantize: ", bits, " bits unsupported (4 or 8)");
    SXB_CHECK(G == 32 || G == 64 || G == 128, "quantize: group size ", G, " unsupported (32, 64 or 128)");
    SXB_CHECK(K % G == 0, "quantize: K = ", K, " is not a multiple of group size ", G);
    SXB_CHECK(reinterpret_cast<uintptr_t>(q) % 4 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0,
              "quantize: w must be 16-byte and q 4-byte aligned");
    const int64_t n_groups = N * (K / G);
    const int64_t blocks = std::min<int64_t>((n_groups * 32 + kThreads - 1) / kThreads, (int64_t)sm_count() * 32);
    auto st = static_cast<cudaStream_t>(stream);
#define SXB_Q(BITS, GG) quantize_kernel<BITS, GG><<<(unsigned)blocks, kThreads, 0, st>>>(w, n_groups, K / G, q, scale, minv, err)
    if (bits == 4) {
        if (G == 32) SXB_Q(4, 32);
        else if (G == 64) SXB_Q(4, 64);
        else SXB_Q(4, 128);
    } else {
        if (G == 32) SXB_Q(8, 32);
        else if (G == 64) SXB_Q(8, 64);
        else SXB_Q(8, 128);
    }
#undef SXB_Q
    SXB_CHECK_LAUNCH("quantize Q", bits, " N=", N, " K=", K, " G=", G);
    return SXB_OK;
}
