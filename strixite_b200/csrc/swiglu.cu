// SwiGLU between an MLP's gate/up and down projections; C ABI twin of kernels/swiglu.hpp:21.
// gu [rows, 2I] = [gate | up] -> h [rows, I]; FP32 math; BF16 rounds as the reference does:
// h = bf16(bf16(silu(g)) * u) (kernels/swiglu.hip:31-36).  Eight (BF16) or four (FP32) columns a thread when the
// rows are whole 16-byte runs, so both operands move as 128-bit accesses.

#include "common.cuh"

namespace sxb {
namespace {

constexpr int kThreads = 256;
constexpr int64_t kMaxElems = 1ll << 40;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<uint16_t> { static constexpr int n = 8; };

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const T *__restrict__ gu, T *__restrict__ h, int64_t n, int64_t I) {
    constexpr int V = VEC ? Vec<T>::n : 1;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * V; i < n; i += (int64_t)gridDim.x * blockDim.x * V) {
        const int64_t r = i / I, j = i % I;
        const T *gp = gu + r * 2 * I + j, *up = gp + I;
        if constexpr (VEC) {
            const uint4 gv = *reinterpret_cast<const uint4 *>(gp), uv = *reinterpret_cast<const uint4 *>(up);
            uint4 hv;
            const T *ge = reinterpret_cast<const T *>(&gv), *ue = reinterpret_cast<const T *>(&uv);
            T *he = reinterpret_cast<T *>(&hv);
#pragma unroll
            for (int e = 0; e < V; ++e)
                store_from_f32(he, e, as_stored<T>(silu_f32(load_as_f32(ge, e))) * load_as_f32(ue, e));
            *reinterpret_cast<uint4 *>(h + i) = hv;
        } else {
            store_from_f32(h, i, as_stored<T>(silu_f32(load_as_f32(gp, 0))) * load_as_f32(up, 0));
        }
    }
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" int sxb_swiglu(const void *gu, void *h, int64_t rows, int64_t I, int act, sxb_stream_t stream) {
    SXB_CHECK(gu != nullptr && h != nullptr, "swiglu: null pointer (gu=", gu, ", h=", h, ")");
    SXB_CHECK(rows >= 1 && I >= 1, "swiglu: rows = ", rows, ", I = ", I, ", both must be >= 1");
    SXB_CHECK(rows <= kMaxElems / I / 2, "swiglu: rows * 2I = ", rows, " * ", 2 * I, " exceeds ", kMaxElems,
              " elements (rows/I swapped?)");
    SXB_CHECK(act_ok(act), "swiglu: unsupported activation dtype ", act);
    const int64_t es = act_bytes(act), n = rows * I;
    SXB_CHECK(apart(h, n * es, gu, 2 * n * es), "swiglu: output h [", h, ", +", n * es, " B) overlaps input gu [", gu,
              ", +", 2 * n * es, " B)");
    const int v = act == SXB_ACT_F32 ? 4 : 8;
    const bool vec = I % v == 0 && aligned16(gu) && aligned16(h);
    const int64_t work = vec ? n / v : n;
    const int64_t blocks = std::min<int64_t>((work + kThreads - 1) / kThreads, (int64_t)sm_count() * 16);
    auto st = static_cast<cudaStream_t>(stream);
    const dim3 grid((unsigned)std::max<int64_t>(blocks, 1));
    if (act == SXB_ACT_F32) {
        if (vec) swiglu_kernel<float, true><<<grid, kThreads, 0, st>>>((const float *)gu, (float *)h, n, I);
        else swiglu_kernel<float, false><<<grid, kThreads, 0, st>>>((const float *)gu, (float *)h, n, I);
    } else {
        if (vec) swiglu_kernel<uint16_t, true><<<grid, kThreads, 0, st>>>((const uint16_t *)gu, (uint16_t *)h, n, I);
        else swiglu_kernel<uint16_t, false><<<grid, kThreads, 0, st>>>((const uint16_t *)gu, (uint16_t *)h, n, I);
    }
    SXB_CHECK_LAUNCH("swiglu ", act_name(act), " rows=", rows, " I=", I);
    return SXB_OK;
}
