// MoE router (top-k + softmax over the picks), the shared expert's gated add, and the error-word readers.
// C ABI twins of kernels/moe_router.hpp in the reference; the arithmetic follows kernels/moe_router.hip:82-111
// (selection order, softmax form) and :129-180 (gated add, residual injection).
//
// Design for sm_100a: one warp per token, kTokensPerCta tokens per CTA.  The E logits of a token live in registers
// (lane l holds experts l, l+32, ...).  A selection round is two warp-wide `redux.sync` reductions on integer keys -
// the maximum of an order-preserving encoding of the lanes' best values, then the minimum expert index among the
// lanes that hold it - instead of five shuffle/compare steps on (value, index) pairs.  Only the lane that owned the
// pick rescans its registers.

#include "router_token.cuh"

#include <algorithm>
#include <mutex>

namespace sxb {

std::string &last_error() {
    static thread_local std::string msg;
    return msg;
}

int fail_check(const char *file, int line, const char *func, const char *cond, const std::string &msg) {
    last_error() = cat(func, " (", file, ":", line, "): check `", cond, "` failed: ", msg);
    return SXB_ERR_CHECK;
}

int fail_cuda(const char *file, int line, const char *func, cudaError_t e, const std::string &msg) {
    last_error() = cat(func, " (", file, ":", line, "): CUDA error ", (int)e, " (", cudaGetErrorName(e), ": ",
                       cudaGetErrorString(e), ") ", msg);
    // Sticky errors poison the context: every later call fails too (the reference's GpuFatalError,
    // common/hip_check.hpp:17-42).
    switch (e) {
        case cudaErrorIllegalAddress:
        case cudaErrorIllegalInstruction:
        case cudaErrorMisalignedAddress:
        case cudaErrorLaunchFailure:
        case cudaErrorHardwareStackError:
        case cudaErrorInvalidAddressSpace:
        case cudaErrorInvalidPc:
        case cudaErrorLaunchTimeout:
        case cudaErrorECCUncorrectable: return SXB_ERR_FATAL;
        default: return SXB_ERR_CUDA;
    }
}

int sm_count() {
    static std::mutex mu;
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

namespace {

constexpr int kLanes = 32;
constexpr int kTokensPerCta = 4;
constexpr int64_t kMaxExperts = 1024;
constexpr int64_t kMaxTopK = 32;
constexpr int64_t kMaxTokens = 0x7fffffff;

template <typename T, int NV>
__global__ void __launch_bounds__(kLanes *kTokensPerCta)
    router_kernel(const T *__restrict__ logits, int64_t ld, int64_t M, int E, int k, const T *__restrict__ shared,
                  int64_t shared_ld, int32_t shared_id, int32_t *__restrict__ ids, float *__restrict__ coef, int A,
                  uint32_t *err) {
    const int lane = threadIdx.x % kLanes;
    const int64_t m = (int64_t)blockIdx.x * kTokensPerCta + threadIdx.x / kLanes;
    if (m >= M) return;  // whole warps leave together
    route_token<T, NV>(logits + m * ld, lane, m, E, k, shared, shared_ld, shared_id, ids + m * A, coef + m * A, A, err);
}

constexpr int kAddThreads = 256;

// y[m, n] = stored(fma(g, s, y)) (+ the H-stream injection).  One thread per column, a CTA per (column slice, row):
// rows are short (N = d) and M small in decode; prefill folds this add into the combine's reduce instead.
template <typename T, bool INJECT>
__global__ void __launch_bounds__(kAddThreads)
    shared_add_kernel(T *__restrict__ y, const T *__restrict__ s, const float *__restrict__ gate_logit, int64_t gate_ld,
                      int64_t N, uint32_t gate_index, T *__restrict__ x, const float *__restrict__ w_in, uint32_t *err) {
    constexpr int kStreams = 4;
    const int64_t m = blockIdx.y;
    const float gl = gate_logit[m * gate_ld];
    const bool ok = isfinite(gl);
    if (!ok && blockIdx.x == 0 && threadIdx.x == 0) raise_error(err, (uint32_t)m, gate_index);
    const float g = ok ? 1.f / (1.f + expf(-gl)) : qnan_f32();
    const int64_t n = (int64_t)blockIdx.x * kAddThreads + threadIdx.x;
    if (n >= N) return;
    const float v = as_stored<T>(fmaf(g, load_as_f32(s, m * N + n), load_as_f32(y, m * N + n)));
    store_from_f32(y, m * N + n, v);
    if constexpr (INJECT) {
        T *xr = x + m * kStreams * N;
#pragma unroll
        for (int st = 0; st < kStreams; ++st)
            store_from_f32(xr, st * N + n, fmaf(w_in[m * kStreams + st], v, load_as_f32(xr, st * N + n)));
    }
}

// kernels/hc.hip:245-252 hc_inject: X[t, s*d + j] += w_in[t, s] * y[t, j] for the H = 4 residual streams, one FP32 rounding
// (fma), then the activation dtype's.  A thread takes one column j of one token and updates its four streams: y is read once.
template <typename T>
__global__ void __launch_bounds__(kAddThreads)
    hc_inject_kernel(T *__restrict__ x, const float *__restrict__ w_in, const T *__restrict__ y, int64_t tokens, int64_t d) {
    constexpr int kStreams = 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < tokens * d; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / d, j = i % d;
        const float v = load_as_f32(y, i);
        T *xr = x + t * kStreams * d;
#pragma unroll
        for (int st = 0; st < kStreams; ++st) store_from_f32(xr, st * d + j, fmaf(w_in[t * kStreams + st], v, load_as_f32(xr, st * d + j)));
    }
}

int read_err_words(const uint32_t *err, uint32_t e[3], const char *fn, const char *what) {
    SXB_CHECK(err != nullptr, fn, "(", what, "): null err");
    SXB_CUDA(cudaMemcpy(e, err, 3 * sizeof(uint32_t), cudaMemcpyDeviceToHost), "reading the error words for ", what);
    return SXB_OK;
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" {

const char *sxb_last_error(void) { return last_error().c_str(); }
const char *sxb_version(void) { return "strix_b200 0.1 sm_100a"; }

int sxb_moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                   int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, int act, uint32_t *err,
                   sxb_stream_t stream) {
    SXB_CHECK(logits != nullptr && ids != nullptr && coef != nullptr && err != nullptr, "moe_router: null pointer (logits=",
              logits, ", ids=", (const void *)ids, ", coef=", (const void *)coef, ", err=", (const void *)err, ")");
    SXB_CHECK(M >= 1 && M <= kMaxTokens, "moe_router: M = ", M, " tokens, expected 1..", kMaxTokens);
    SXB_CHECK(E >= 1 && E <= kMaxExperts, "moe_router: E = ", E, " experts, expected 1..", kMaxExperts);
    SXB_CHECK(k >= 1 && k <= E && k <= kMaxTopK, "moe_router: k = ", k, ", expected 1..min(E = ", E, ", ", kMaxTopK, ")");
    SXB_CHECK(ld >= E, "moe_router: logits row stride ld = ", ld, " < E = ", E);
    if (shared_logit != nullptr) {
        SXB_CHECK(shared_ld >= 1, "moe_router: shared_ld = ", shared_ld, ", expected >= 1");
        SXB_CHECK(shared_id >= 0, "moe_router: shared_id = ", shared_id, ", expected >= 0 (its expert row block)");
    }
    SXB_CHECK((const void *)ids != (const void *)coef, "moe_router: ids and coef are the same buffer");
    SXB_CHECK(act_ok(act), "moe_router: unsupported activation dtype ", act);
    const int A = (int)k + (shared_logit != nullptr ? 1 : 0);
    const dim3 grid((unsigned)((M + kTokensPerCta - 1) / kTokensPerCta)), block(kLanes * kTokensPerCta);
    auto st = static_cast<cudaStream_t>(stream);
#define SXB_ROUTER(T, NV)                                                                                         \
    router_kernel<T, NV><<<grid, block, 0, st>>>(static_cast<const T *>(logits), ld, M, (int)E, (int)k,            \
                                                 static_cast<const T *>(shared_logit), shared_ld, shared_id, ids, \
                                                 coef, A, err)
#define SXB_ROUTER_NV(T)                 \
    if (E <= 128) SXB_ROUTER(T, 4);      \
    else if (E <= 256) SXB_ROUTER(T, 8); \
    else if (E <= 512) SXB_ROUTER(T, 16); \
    else SXB_ROUTER(T, 32)
    if (act == SXB_ACT_F32) {
        SXB_ROUTER_NV(float);
    } else {
        SXB_ROUTER_NV(uint16_t);
    }
#undef SXB_ROUTER_NV
#undef SXB_ROUTER
    SXB_CHECK_LAUNCH("moe_router ", act_name(act), " M=", M, " E=", E, " k=", k, shared_logit ? " +shared" : "");
    return SXB_OK;
}

int sxb_report_router_error(const uint32_t e[3], const char *what) {
    if (e[0] == 0) return SXB_OK;
    last_error() = cat(what, ": non-finite router logit at token ", e[1], ", expert ", e[2],
                       " (E = the shared-expert gate); that token's ids are -1 and its coefficients NaN");
    return SXB_ERR_DATA;
}

int sxb_check_router_error(const uint32_t *err, const char *what) {
    uint32_t e[3];
    if (int rc = read_err_words(err, e, "check_router_error", what)) return rc;
    return sxb_report_router_error(e, what);
}

int sxb_report_expert_error(const uint32_t e[3], const char *what) {
    if (e[0] == 0) return SXB_OK;
    last_error() = cat(what, ": expert id ", (int32_t)e[1], " at slot ", e[2],
                       " (token * A + a) is out of range; outputs for that token are NaN");
    return SXB_ERR_DATA;
}

int sxb_check_expert_error(const uint32_t *err, const char *what) {
    uint32_t e[3];
    if (int rc = read_err_words(err, e, "check_expert_error", what)) return rc;
    return sxb_report_expert_error(e, what);
}

static int shared_add_impl(const char *fn, void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M,
                           int64_t N, uint32_t gate_index, void *x, const float *w_in, int64_t H, bool inject, int act,
                           uint32_t *err, sxb_stream_t stream) {
    SXB_CHECK(y != nullptr && s != nullptr && gate_logit != nullptr && err != nullptr, fn, ": null pointer (y=", y,
              ", s=", s, ", gate_logit=", (const void *)gate_logit, ", err=", (const void *)err, ")");
    SXB_CHECK(!inject || (x != nullptr && w_in != nullptr), fn, ": null pointer (x=", x, ", w_in=", (const void *)w_in, ")");
    SXB_CHECK(M >= 1 && M <= 65535, fn, ": M = ", M, " tokens, expected 1..65535 (grid.y)");
    SXB_CHECK(N >= 1 && N <= (1ll << 24), fn, ": N = ", N, ", expected 1..2^24");
    SXB_CHECK(!inject || H == 4, fn, ": H = ", H, " streams, expected 4");
    SXB_CHECK(gate_ld >= 1, fn, ": gate_ld = ", gate_ld, ", expected >= 1");
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    const int64_t ybytes = M * N * act_bytes(act), xbytes = M * H * N * act_bytes(act);
    SXB_CHECK(apart(y, ybytes, s, ybytes), fn, ": s [", s, ", +", ybytes, " B) overlaps y [", y, ", +", ybytes, " B)");
    if (inject)
        SXB_CHECK(apart(x, xbytes, y, ybytes) && apart(x, xbytes, s, ybytes), fn, ": x [", x, ", +", xbytes,
                  " B) overlaps y [", y, "] or s [", s, "] (", ybytes, " B each)");
    const dim3 grid((unsigned)((N + kAddThreads - 1) / kAddThreads), (unsigned)M), block(kAddThreads);
    auto st = static_cast<cudaStream_t>(stream);
    if (act == SXB_ACT_F32) {
        if (inject)
            shared_add_kernel<float, true><<<grid, block, 0, st>>>((float *)y, (const float *)s, gate_logit, gate_ld, N,
                                                                   gate_index, (float *)x, w_in, err);
        else
            shared_add_kernel<float, false><<<grid, block, 0, st>>>((float *)y, (const float *)s, gate_logit, gate_ld, N,
                                                                    gate_index, nullptr, nullptr, err);
    } else {
        if (inject)
            shared_add_kernel<uint16_t, true><<<grid, block, 0, st>>>((uint16_t *)y, (const uint16_t *)s, gate_logit,
                                                                      gate_ld, N, gate_index, (uint16_t *)x, w_in, err);
        else
            shared_add_kernel<uint16_t, false><<<grid, block, 0, st>>>((uint16_t *)y, (const uint16_t *)s, gate_logit,
                                                                       gate_ld, N, gate_index, nullptr, nullptr, err);
    }
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), " M=", M, " N=", N);
    return SXB_OK;
}

int sxb_hc_inject(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, int act, sxb_stream_t stream) {
    const char *fn = "hc_inject";
    SXB_CHECK(x != nullptr && w_in != nullptr && y != nullptr, fn, ": null pointer (x=", x, ", w_in=", (const void *)w_in, ", y=", y, ")");
    SXB_CHECK(H == 4, fn, ": H = ", H, " streams, expected 4");
    SXB_CHECK(T >= 1 && d >= 1 && d <= (1 << 20) && T <= (1ll << 40) / (H * d), fn, ": T = ", T, ", d = ", d);
    SXB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SXB_CHECK(apart(x, T * H * d * act_bytes(act), y, T * d * act_bytes(act)), fn, ": y overlaps X");
    const unsigned blocks = (unsigned)std::min<int64_t>((T * d + kAddThreads - 1) / kAddThreads, (int64_t)sm_count() * 16);
    auto st = static_cast<cudaStream_t>(stream);
    if (act == SXB_ACT_F32) hc_inject_kernel<float><<<blocks, kAddThreads, 0, st>>>((float *)x, w_in, (const float *)y, T, d);
    else hc_inject_kernel<uint16_t><<<blocks, kAddThreads, 0, st>>>((uint16_t *)x, w_in, (const uint16_t *)y, T, d);
    SXB_CHECK_LAUNCH(fn, " ", act_name(act), " T=", T, " d=", d);
    return SXB_OK;
}

int sxb_moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                       uint32_t gate_index, int act, uint32_t *err, sxb_stream_t stream) {
    return shared_add_impl("moe_shared_add", y, s, gate_logit, gate_ld, M, N, gate_index, nullptr, nullptr, 4, false,
                           act, err, stream);
}

int sxb_moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                              uint32_t gate_index, void *x, const float *w_in, int64_t H, int act, uint32_t *err,
                              sxb_stream_t stream) {
    return shared_add_impl("moe_shared_add_inject", y, s, gate_logit, gate_ld, M, N, gate_index, x, w_in, H, true, act,
                           err, stream);
}

}  // extern "C"
