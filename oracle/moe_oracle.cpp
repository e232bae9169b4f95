// CPU oracle for the quantized MoE FFN path.  TEST INFRASTRUCTURE ONLY: nothing in the
// shipped library links, loads or calls this file; tests, the smoke check and the CPU
// baseline leg of the benchmark are its only users.
//
// It restates, as plain multi-threaded C++, the arithmetic that the reference documents
// for this path.  Each function names the reference file:line it follows.  The reference
// ships no CPU implementation and no golden vectors for these kernels, so parity with the
// reference's device code is pinned only for the quantizers (checked bit-for-bit against
// the reference's own formats/q4.cpp and formats/q8.cpp compiled by oracle/Makefile);
// for router / pack / expert math parity is "unpinned": it rests on the header prose and
// kernel sources cited below.  PARITY UNPINNED for those parts.
//
// Conventions: BF16 values travel as raw uint16_t bits; "act" 0 = F32, 1 = BF16
// (kernels/norm.hpp:20).  Expert weights are stacked [E*N, K] (kernels/linear_q4.hpp:32-35).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

namespace {

// common/bf16.hpp:14-27 - round to nearest even, non-finite preserved.
inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x0040u : 0u));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float as_stored(float v, int act) { return act == 1 ? bf16_to_f32(f32_to_bf16(v)) : v; }
inline float load_act(const void *p, int64_t i, int act) {
    return act == 1 ? bf16_to_f32(static_cast<const uint16_t *>(p)[i]) : static_cast<const float *>(p)[i];
}
inline void store_act(void *p, int64_t i, float v, int act) {
    if (act == 1) static_cast<uint16_t *>(p)[i] = f32_to_bf16(v);
    else static_cast<float *>(p)[i] = v;
}
inline float qnan() { return std::numeric_limits<float>::quiet_NaN(); }
// kernels/swiglu.hip:22 - silu(v) = v / (1 + expf(-v)), all in FP32.
inline float silu(float v) { return v / (1.0f + std::exp(-v)); }

int n_threads(int requested) {
    if (requested > 0) return requested;
    unsigned hc = std::thread::hardware_concurrency();
    return hc ? (int)hc : 1;
}

// Dynamic work queue over [0, n): every task index is taken exactly once.
void parallel_for(int64_t n, int threads, const std::function<void(int64_t)> &fn) {
    threads = (int)std::min<int64_t>(n_threads(threads), std::max<int64_t>(n, 1));
    if (threads <= 1) {
        for (int64_t i = 0; i < n; ++i) fn(i);
        return;
    }
    std::atomic<int64_t> next{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([&] {
            for (int64_t i; (i = next.fetch_add(1)) < n;) fn(i);
        });
    for (auto &th : pool) th.join();
}

struct QView {
    const uint8_t *q;
    const uint16_t *scale, *minv;
    int64_t N, K, G;
    int bits;  // 4 or 8
};

inline int code_at(const QView &w, int64_t row, int64_t k) {
    if (w.bits == 8) return w.q[row * w.K + k];
    return (w.q[(row * w.K + k) / 2] >> ((k & 1) ? 4 : 0)) & 0xF;  // formats/q4.hpp:5 low nibble = even k
}

// IEEE binary16 <-> double, round to nearest even, subnormals kept (what the device's packed-half arithmetic does).
double f16_bits_to_double(uint16_t h) {
    const int sign = h >> 15, e = (h >> 10) & 0x1F, f = h & 0x3FF;
    double v;
    if (e == 0) v = std::ldexp((double)f, -24);
    else if (e == 31) v = f ? std::numeric_limits<double>::quiet_NaN() : std::numeric_limits<double>::infinity();
    else v = std::ldexp((double)(f | 0x400), e - 25);
    return sign ? -v : v;
}
uint16_t double_to_f16_bits(double v) {
    const uint16_t sign = std::signbit(v) ? 0x8000 : 0;
    v = std::fabs(v);
    if (std::isnan(v)) return sign | 0x7E00;
    if (v >= 65520.0) return sign | 0x7C00;  // rounds to infinity
    if (v < std::ldexp(1.0, -25)) return sign;  // below half the smallest subnormal (ties to even: 0)
    int e;
    std::frexp(v, &e);                  // v = m * 2^e, m in [0.5, 1)
    int exp = e - 1;                    // v = 1.xxx * 2^exp
    if (exp < -14) exp = -14;           // subnormal: fixed exponent
    const double scaled = std::ldexp(v, 10 - exp);  // units of the last place
    double r = std::nearbyint(scaled);  // half to even
    int64_t q = (int64_t)r;
    if (exp == -14 && q < 0x400) return sign | (uint16_t)q;  // subnormal (or rounds up into the first normal below)
    if (q >= 0x800) q >>= 1, ++exp;     // the rounding carried into the next binade
    if (exp > 15) return sign | 0x7C00;
    return sign | (uint16_t)(((exp + 15) << 10) | (q & 0x3FF));
}
inline float round_f16(double v) { return (float)f16_bits_to_double(double_to_f16_bits(v)); }
// Round toward zero to binary16: the largest-magnitude F16 value not beyond v (what the reference's staging of BF16
// activations does, kernels/moe_grouped.hip:29-32; exact for BF16 inputs in F16's normal range either way).
inline float trunc_f16(double v) {
    const double r = f16_bits_to_double(double_to_f16_bits(v));
    if (std::isnan(r) || std::fabs(r) <= std::fabs(v)) return (float)r;
    if (std::isinf(r)) return std::signbit(v) ? -65504.0f : 65504.0f;  // nearest rounded past the largest finite value
    const uint16_t bits = double_to_f16_bits(v);
    return (float)f16_bits_to_double((uint16_t)(bits - 1));  // one step toward zero (same sign, smaller magnitude)
}
// Activation staging of the matrix-unit path: mode 0 keeps the value, 1 rounds to F16 (nearest even), 2 toward zero.
inline float stage_f16(float v, int mode) { return mode == 0 ? v : mode == 1 ? round_f16(v) : trunc_f16(v); }

// One dequantized row.
//   f16 == false: the FP32 values of formats/q4.cpp:121-134 / formats/q8.cpp:117-127 - code * scale, then + min, each
//                 rounded separately (no FMA contraction): the weights of the exact / vector-unit paths.
//   f16 == true:  the matrix-unit path's operand (kernels/moe_grouped.hpp:32-33, kernels/wmma_gemm.hpp:116-129):
//                 scale and min converted to F16, then f16(code * scale + min) with ONE rounding (an F16 fma).
void dequant_row(const QView &w, int64_t row, float *out, bool f16 = false) {
    const int64_t groups = w.K / w.G;
    for (int64_t g = 0; g < groups; ++g) {
        const float s = bf16_to_f32(w.scale[row * groups + g]), m = bf16_to_f32(w.minv[row * groups + g]);
        if (f16) {
            const double sh = round_f16(s), mh = round_f16(m);
            for (int64_t i = 0; i < w.G; ++i) {
                const int64_t k = g * w.G + i;
                out[k] = round_f16((double)code_at(w, row, k) * sh + mh);  // exact in double, then one rounding
            }
            continue;
        }
        for (int64_t i = 0; i < w.G; ++i) {
            const int64_t k = g * w.G + i;
            out[k] = (float)code_at(w, row, k) * s + m;  // two roundings: built with -ffp-contract=off
        }
    }
}

inline double dot_f32(const float *a, const float *b, int64_t n) {
    double acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
    int64_t i = 0;
    for (; i + 4 <= n; i += 4) {
        acc0 += (double)a[i] * (double)b[i];
        acc1 += (double)a[i + 1] * (double)b[i + 1];
        acc2 += (double)a[i + 2] * (double)b[i + 2];
        acc3 += (double)a[i + 3] * (double)b[i + 3];
    }
    for (; i < n; ++i) acc0 += (double)a[i] * (double)b[i];
    return (acc0 + acc1) + (acc2 + acc3);
}

// Slots of ids [S] bucketed by expert, stable in slot order; invalid ids go to bucket E.
void bucket_slots(const int32_t *ids, int64_t S, int64_t E, std::vector<std::vector<int64_t>> &buckets) {
    buckets.assign((size_t)E + 1, {});
    for (int64_t s = 0; s < S; ++s) {
        const int32_t id = ids[s];
        buckets[(size_t)((id < 0 || id >= E) ? E : id)].push_back(s);
    }
}

// kernels/linear_q4.hip:166-173 - first writer wins.
void flag_error(uint32_t *err, uint32_t a, uint32_t b) {
    if (err && err[0] == 0u) err[0] = 1u, err[1] = a, err[2] = b;
}

constexpr int kRowBlock = 16;

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------
// Quantizers: formats/q4.cpp:44-88 (Q4) and formats/q8.cpp:43-82 (Q8).
//   s = bf16((max - min) / levels), m = bf16(min), code = clamp(nearbyint((w - m) / s), 0, levels)
//   with s == 0 -> code 0; all FP32.  Returns 0, or 1 on a bad shape / non-finite input.
int orc_quantize(const float *w, int64_t N, int64_t K, int64_t G, int bits, uint8_t *q, uint16_t *scale,
                 uint16_t *minv) {
    if (!w || N < 1 || K < 1 || !(G == 32 || G == 64 || G == 128) || K % G != 0 || !(bits == 4 || bits == 8)) return 1;
    const float levels = bits == 4 ? 15.0f : 255.0f;
    const int64_t groups = K / G;
    std::memset(q, 0, (size_t)(bits == 4 ? N * K / 2 : N * K));
    std::atomic<int> bad{0};
    parallel_for(N, 0, [&](int64_t n) {
        for (int64_t g = 0; g < groups; ++g) {
            const float *grp = w + n * K + g * G;
            float lo = grp[0], hi = grp[0];
            for (int64_t i = 0; i < G; ++i) {
                if (!std::isfinite(grp[i])) bad = 1;
                lo = std::fmin(lo, grp[i]);
                hi = std::fmax(hi, grp[i]);
            }
            const uint16_t s_bits = f32_to_bf16((hi - lo) / levels), m_bits = f32_to_bf16(lo);
            const float s = bf16_to_f32(s_bits), m = bf16_to_f32(m_bits);
            scale[n * groups + g] = s_bits;
            minv[n * groups + g] = m_bits;
            for (int64_t i = 0; i < G; ++i) {
                int code = 0;
                if (s > 0.0f) {
                    const float r = std::nearbyint((grp[i] - m) / s);  // half to even (default rounding mode)
                    code = (int)std::fmin(std::fmax(r, 0.0f), levels);
                }
                const int64_t k = g * G + i;
                if (bits == 4) q[(n * K + k) / 2] |= (uint8_t)(code << ((k & 1) ? 4 : 0));
                else q[n * K + k] = (uint8_t)code;
            }
        }
    });
    return bad.load();
}

void orc_dequantize(const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K, int64_t G,
                    int bits, float *w) {
    const QView v{q, scale, minv, N, K, G, bits};
    parallel_for(N, 0, [&](int64_t n) { dequant_row(v, n, w + n * K); });
}

// ---------------------------------------------------------------------------------------
// Router: kernels/moe_router.hpp:11-23, kernels/moe_router.hip:43-111.
//   k picks, larger logit first, a tie to the lower index; coef_j = expf(l_j - l_top) / sum,
//   the sum formed by a 32-lane xor butterfly over lanes 0..k-1 (others contribute 0);
//   optional slot k: id = shared_id, coef = 1 / (1 + expf(-gate)).
//   A non-finite logit fails its token: ids -1, coef NaN, err = {1, token, smallest bad index}.
void orc_moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                    int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, int act, uint32_t *err) {
    const int64_t A = k + (shared_logit ? 1 : 0);
    std::vector<float> v((size_t)E);
    for (int64_t m = 0; m < M; ++m) {
        int64_t bad = -1;
        for (int64_t e = 0; e < E; ++e) {
            v[(size_t)e] = load_act(logits, m * ld + e, act);
            if (!std::isfinite(v[(size_t)e]) && bad < 0) bad = e;
        }
        float sl = 0.f;
        if (shared_logit) {
            sl = load_act(shared_logit, m * shared_ld, act);
            if (!std::isfinite(sl) && bad < 0) bad = E;
        }
        if (bad >= 0) {
            flag_error(err, (uint32_t)m, (uint32_t)bad);
            for (int64_t a = 0; a < A; ++a) ids[m * A + a] = -1, coef[m * A + a] = qnan();
            continue;
        }
        float pick_v[32];
        int32_t pick_i[32];
        for (int64_t r = 0; r < k; ++r) {
            int64_t best = -1;
            for (int64_t e = 0; e < E; ++e)
                if (best < 0 || v[(size_t)e] > v[(size_t)best]) best = e;  // strict >: the lower index keeps a tie
            pick_v[r] = v[(size_t)best];
            pick_i[r] = (int32_t)best;
            v[(size_t)best] = -std::numeric_limits<float>::infinity();
        }
        float lane[32];
        for (int l = 0; l < 32; ++l) lane[l] = l < k ? std::exp(pick_v[l] - pick_v[0]) : 0.f;
        float sum[32], tmp[32];
        std::memcpy(sum, lane, sizeof(sum));
        for (int off = 16; off > 0; off >>= 1) {
            for (int l = 0; l < 32; ++l) tmp[l] = sum[l] + sum[l ^ off];
            std::memcpy(sum, tmp, sizeof(sum));
        }
        for (int64_t r = 0; r < k; ++r) ids[m * A + r] = pick_i[r], coef[m * A + r] = lane[r] / sum[r];
        if (shared_logit) ids[m * A + k] = shared_id, coef[m * A + k] = 1.0f / (1.0f + std::exp(-sl));
    }
}

// ---------------------------------------------------------------------------------------
// Pack: kernels/moe_grouped.hip:89-92,136-188.  Counting sort of the S = M*A slots by expert
// id into E + 1 buckets (bucket E = ids outside [0, E)); offsets = exclusive scan of the
// counts, offsets[E+1] = S.  The reference leaves the order inside a bucket to its atomics;
// here it is ascending slot index (stable), which the CUDA pack reproduces.
// err = {1, id, slot} for the first invalid slot in slot order.
void orc_moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, int32_t *offsets, int32_t *slots,
                          uint32_t *err) {
    const int64_t S = M * A;
    std::vector<std::vector<int64_t>> b;
    bucket_slots(ids, S, E, b);
    int64_t pos = 0;
    for (int64_t e = 0; e <= E; ++e) {
        offsets[e] = (int32_t)pos;
        for (int64_t s : b[(size_t)e]) slots[pos++] = (int32_t)s;
    }
    offsets[E + 1] = (int32_t)pos;
    if (!b[(size_t)E].empty()) flag_error(err, (uint32_t)ids[b[(size_t)E][0]], (uint32_t)b[(size_t)E][0]);
}

// ---------------------------------------------------------------------------------------
// Dense linear: kernels/linear_q4.hpp:1-30, kernels/linear_q8.hpp:1-14.
//   y[M, N] = x[M, K] * dequant(W)^T, accumulated here in double and cast to FP32 (the
//   kernels accumulate in FP32; only the summation order differs), one rounding at the store.
void orc_linear_q(const void *x, int act, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N,
                  int64_t K, int64_t G, int bits, void *y, int out_act, int64_t M, int threads, int w_f16) {
    const QView w{q, scale, minv, N, K, G, bits};
    std::vector<float> xf((size_t)(M * K));
    for (int64_t i = 0; i < M * K; ++i) xf[(size_t)i] = load_act(x, i, act);
    const int64_t blocks = (N + kRowBlock - 1) / kRowBlock;
    parallel_for(blocks, threads, [&](int64_t b) {
        std::vector<float> row((size_t)K);
        for (int64_t n = b * kRowBlock; n < std::min(N, (b + 1) * kRowBlock); ++n) {
            dequant_row(w, n, row.data(), w_f16 != 0);
            for (int64_t m = 0; m < M; ++m) store_act(y, m * N + n, (float)dot_f32(&xf[(size_t)(m * K)], row.data(), K), out_act);
        }
    });
}

// ---------------------------------------------------------------------------------------
// SwiGLU: kernels/swiglu.hpp:6-10, kernels/swiglu.hip:24-37.
//   gu [rows, 2I] = [gate | up] -> h [rows, I]; BF16: h = bf16(bf16(silu(g)) * u).
void orc_swiglu(const void *gu, void *h, int64_t rows, int64_t I, int act) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < I; ++j) {
            const float g = load_act(gu, r * 2 * I + j, act), u = load_act(gu, r * 2 * I + I + j, act);
            store_act(h, r * I + j, as_stored(silu(g), act) * u, act);
        }
}

// ---------------------------------------------------------------------------------------
// Experts gather: kernels/linear_q4.hpp:36-41, kernels/linear_q4.hip:215-237 (plain) and
// :248-276 (SwiGLU epilogue).  y[m, a, :] = x[m, :] * W[ids[m, a]]^T.
//   swiglu_mode 0: plain gather, y [M, A, N].
//   swiglu_mode 1 (decode semantics, kernels/linear_q4.hip:272-274): g, u rounded as stored,
//                 h = stored(stored(silu(g)) * u), h [M, A, N/2].
//   swiglu_mode 2 (grouped matrix-unit semantics, kernels/moe_grouped.hip:508-524):
//                 h = stored(silu(g_f32) * u_f32), one rounding.
//   w_f16: the weights are the matrix-unit path's F16 operand (see dequant_row) instead of the FP32 dequantization.
//   x_f16: the activations as that path stages them: 0 as they are, 1 F16 to nearest, 2 F16 toward zero
//          (kernels/moe_grouped.hip:29-32).
// An id outside [0, E): err = {1, id, slot}, that slot's outputs NaN.
void orc_experts_gather(const void *x, int act, const uint8_t *q, const uint16_t *scale, const uint16_t *minv,
                        int64_t Ntot, int64_t K, int64_t G, int bits, int64_t E, const int32_t *ids, int64_t M,
                        int64_t A, void *y, int swiglu_mode, uint32_t *err, int threads, int w_f16, int x_f16) {
    const QView w{q, scale, minv, Ntot, K, G, bits};
    const int64_t N = Ntot / E, S = M * A, I = N / 2, out_cols = swiglu_mode ? I : N;
    std::vector<float> xf((size_t)(M * K));
    for (int64_t i = 0; i < M * K; ++i) xf[(size_t)i] = stage_f16(load_act(x, i, act), x_f16);
    std::vector<std::vector<int64_t>> b;
    bucket_slots(ids, S, E, b);
    for (int64_t s : b[(size_t)E]) {
        flag_error(err, (uint32_t)ids[s], (uint32_t)s);
        for (int64_t c = 0; c < out_cols; ++c) store_act(y, s * out_cols + c, qnan(), act);
    }
    const int64_t blocks_per_e = (out_cols + kRowBlock - 1) / kRowBlock;
    parallel_for(E * blocks_per_e, threads, [&](int64_t task) {
        const int64_t e = task / blocks_per_e, blk = task % blocks_per_e;
        const auto &slots = b[(size_t)e];
        if (slots.empty()) return;
        std::vector<float> row((size_t)K), row2((size_t)K);
        for (int64_t c = blk * kRowBlock; c < std::min(out_cols, (blk + 1) * kRowBlock); ++c) {
            dequant_row(w, e * N + c, row.data(), w_f16 != 0);
            if (swiglu_mode) dequant_row(w, e * N + I + c, row2.data(), w_f16 != 0);
            for (int64_t s : slots) {
                const float *xr = &xf[(size_t)((s / A) * K)];
                const float g = (float)dot_f32(xr, row.data(), K);
                if (!swiglu_mode) {
                    store_act(y, s * N + c, g, act);
                    continue;
                }
                const float u = (float)dot_f32(xr, row2.data(), K);
                float hv;
                if (swiglu_mode == 1) hv = as_stored(silu(as_stored(g, act)), act) * as_stored(u, act);
                else hv = silu(g) * u;
                store_act(y, s * I + c, hv, act);
            }
        }
    });
}

// ---------------------------------------------------------------------------------------
// Experts combine: kernels/linear_q4.hpp:38-39, kernels/linear_q4.hip:281-322.
//   y[m, :] = sum_a coef[m, a] * (h[m, a, :] * W[ids[m, a]]^T), one rounding at the store.
// Each per-slot dot is formed in double and cast to FP32; the sum over a runs in slot order
// in double.  partial_out (optional, [M*A, N] FP32) receives the per-slot dots
// (kernels/moe_grouped.hpp:84-87).  partial_bf16: every per-slot dot is rounded to BF16 before the sum, as the
// reference's matrix-unit path stores them (kernels/moe_grouped.hip:47-57); x_f16 as in orc_experts_gather.
// Any invalid id of a token: err, its whole y row NaN.
void orc_experts_combine(const void *h, int act, const uint8_t *q, const uint16_t *scale, const uint16_t *minv,
                         int64_t Ntot, int64_t K, int64_t G, int bits, int64_t E, const int32_t *ids,
                         const float *coef, int64_t M, int64_t A, void *y, int out_act, float *partial_out,
                         uint32_t *err, int threads, int w_f16, int x_f16, int partial_bf16) {
    const QView w{q, scale, minv, Ntot, K, G, bits};
    const int64_t N = Ntot / E, S = M * A;
    std::vector<float> hf((size_t)(S * K));
    for (int64_t i = 0; i < S * K; ++i) hf[(size_t)i] = stage_f16(load_act(h, i, act), x_f16);
    std::vector<float> local;
    float *partial = partial_out;
    if (!partial) {
        local.assign((size_t)(S * N), 0.f);
        partial = local.data();
    }
    std::vector<std::vector<int64_t>> b;
    bucket_slots(ids, S, E, b);
    for (int64_t s : b[(size_t)E]) {
        flag_error(err, (uint32_t)ids[s], (uint32_t)s);
        for (int64_t n = 0; n < N; ++n) partial[s * N + n] = qnan();
    }
    const int64_t blocks_per_e = (N + kRowBlock - 1) / kRowBlock;
    parallel_for(E * blocks_per_e, threads, [&](int64_t task) {
        const int64_t e = task / blocks_per_e, blk = task % blocks_per_e;
        const auto &slots = b[(size_t)e];
        if (slots.empty()) return;
        std::vector<float> row((size_t)K);
        for (int64_t n = blk * kRowBlock; n < std::min(N, (blk + 1) * kRowBlock); ++n) {
            dequant_row(w, e * N + n, row.data(), w_f16 != 0);
            for (int64_t s : slots) {
                const float p = (float)dot_f32(&hf[(size_t)(s * K)], row.data(), K);
                partial[s * N + n] = partial_bf16 ? bf16_to_f32(f32_to_bf16(p)) : p;  // kernels/moe_grouped.hip:47-57
            }
        }
    });
    parallel_for(M, threads, [&](int64_t m) {
        bool ok = true;
        for (int64_t a = 0; a < A; ++a) ok = ok && ids[m * A + a] >= 0 && ids[m * A + a] < E;
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0;
            for (int64_t a = 0; a < A; ++a) acc += (double)coef[m * A + a] * (double)partial[(m * A + a) * N + n];
            store_act(y, m * N + n, ok ? (float)acc : qnan(), out_act);
        }
    });
}

// ---------------------------------------------------------------------------------------
// Shared expert's gated add: kernels/moe_router.hpp:44-54, kernels/moe_router.hip:129-145.
//   y[m, :] = stored(y + sigmoid(gate_logit[m * gate_ld]) * s); non-finite gate -> NaN row,
//   err = {1, token, gate_index}.
void orc_moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                        uint32_t gate_index, int act, uint32_t *err) {
    for (int64_t m = 0; m < M; ++m) {
        const float gl = gate_logit[m * gate_ld];
        const bool ok = std::isfinite(gl);
        if (!ok) flag_error(err, (uint32_t)m, gate_index);
        const float g = ok ? 1.f / (1.f + std::exp(-gl)) : qnan();
        for (int64_t n = 0; n < N; ++n) {
            // `y + g * s` in the device source; the reference's device compiler contracts it into one fma
            store_act(y, m * N + n, std::fma(g, load_act(s, m * N + n, act), load_act(y, m * N + n, act)), act);
        }
    }
}

// kernels/moe_router.hpp:56-63, kernels/moe_router.hip:154-180: the add above on the stored y,
// then x[m, st*N + n] = stored(fma(w_in[m, st], y, x)) for the H = 4 residual streams.
void orc_moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                               uint32_t gate_index, void *x, const float *w_in, int64_t H, int act, uint32_t *err) {
    orc_moe_shared_add(y, s, gate_logit, gate_ld, M, N, gate_index, act, err);
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            const float v = load_act(y, m * N + n, act);
            for (int64_t st = 0; st < H; ++st) {
                const int64_t i = m * H * N + st * N + n;
                store_act(x, i, std::fma(w_in[m * H + st], v, load_act(x, i, act)), act);
            }
        }
}

// Host threads the oracle uses when asked for "all" (threads <= 0).
int orc_hardware_threads() { return n_threads(0); }

}  // extern "C"
