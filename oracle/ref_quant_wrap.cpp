// C entry points over the REFERENCE's own quantizers (formats/q4.cpp, formats/q8.cpp), which
// oracle/Makefile compiles unchanged from the reference checkout into oracle/_ref/.  Test
// infrastructure only: used to pin the oracle's and the CUDA quantizers' outputs bit for bit.
#include "formats/q4.hpp"
#include "formats/q8.hpp"

#include <cstdint>
#include <cstring>
#include <exception>

extern "C" {

// bits 4: q holds N*K/2 bytes; bits 8: N*K bytes.  Returns 0, or 1 if the reference threw.
int ref_quantize(const float *w, int64_t N, int64_t K, int64_t G, int bits, uint8_t *q, uint16_t *scale,
                 uint16_t *minv) {
    try {
        if (bits == 4) {
            const strix::Q4Weight r = strix::quantize_q4(w, N, K, G);
            std::memcpy(q, r.q.data(), r.q.size());
            std::memcpy(scale, r.scale.data(), 2 * r.scale.size());
            std::memcpy(minv, r.minv.data(), 2 * r.minv.size());
        } else {
            const strix::Q8Weight r = strix::quantize_q8(w, N, K, G);
            std::memcpy(q, r.q.data(), r.q.size());
            std::memcpy(scale, r.scale.data(), 2 * r.scale.size());
            std::memcpy(minv, r.minv.data(), 2 * r.minv.size());
        }
    } catch (const std::exception &) {
        return 1;
    }
    return 0;
}

int ref_dequantize(const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K, int64_t G,
                   int bits, float *w) {
    try {
        const size_t groups = (size_t)(N * (K / G));
        if (bits == 4) {
            strix::Q4Weight r;
            r.N = N, r.K = K, r.G = G;
            r.q.assign(q, q + N * K / 2);
            r.scale.assign(scale, scale + groups);
            r.minv.assign(minv, minv + groups);
            const auto out = strix::dequantize_q4(r);
            std::memcpy(w, out.data(), 4 * out.size());
        } else {
            strix::Q8Weight r;
            r.N = N, r.K = K, r.G = G;
            r.q.assign(q, q + N * K);
            r.scale.assign(scale, scale + groups);
            r.minv.assign(minv, minv + groups);
            const auto out = strix::dequantize_q8(r);
            std::memcpy(w, out.data(), 4 * out.size());
        }
    } catch (const std::exception &) {
        return 1;
    }
    return 0;
}

// formats/q4.hpp:55 / formats/q8.hpp:46 to_chunk_major: q holds the same number of bytes as the source, scale / minv N * (K / G).
int ref_to_chunk_major(const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K, int64_t G, int bits,
                       uint8_t *qo, uint16_t *so, uint16_t *mo) {
    try {
        const size_t groups = (size_t)(N * (K / G));
        if (bits == 4) {
            strix::Q4Weight r;
            r.N = N, r.K = K, r.G = G;
            r.q.assign(q, q + N * K / 2), r.scale.assign(scale, scale + groups), r.minv.assign(minv, minv + groups);
            const strix::Q4ChunkMajor c = strix::to_chunk_major(r, "ref_to_chunk_major");
            std::memcpy(qo, c.q.data(), c.q.size()), std::memcpy(so, c.scale.data(), 2 * c.scale.size()), std::memcpy(mo, c.minv.data(), 2 * c.minv.size());
        } else {
            strix::Q8Weight r;
            r.N = N, r.K = K, r.G = G;
            r.q.assign(q, q + N * K), r.scale.assign(scale, scale + groups), r.minv.assign(minv, minv + groups);
            const strix::Q8ChunkMajor c = strix::to_chunk_major(r, "ref_to_chunk_major");
            std::memcpy(qo, c.q.data(), c.q.size()), std::memcpy(so, c.scale.data(), 2 * c.scale.size()), std::memcpy(mo, c.minv.data(), 2 * c.minv.size());
        }
    } catch (const std::exception &) {
        return 1;
    }
    return 0;
}

}  // extern "C"
