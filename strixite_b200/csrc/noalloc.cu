// sxb_linear_q4_experts_combine_grouped_noalloc: the grouped down projection + combine for hosts that cannot hand the
// library a scratch buffer.  It is sxb_linear_q4_experts_combine_grouped with one argument fewer: the per-slot dots
// ("partial", M*A*N FP32) live in an array that is part of the library image instead of in caller memory.
//
// Who needs this: an engine that sized its device memory plan at start-up and gave every byte to weights and K/V pages
// has nothing left to carve a scratch buffer from, and a decode loop cannot call cudaMalloc either - it synchronizes the
// device and would stall the very stream the step is running on.  Such callers still own x / h / y (the model's
// activations); what they lack is the few megabytes of scratch between the two kernels of the combine.
//
// The array's name below is a host-side handle, not a device address: launching a kernel with `g_partial` itself as
// an argument would hand it a host pointer.  The device address is looked up once per device with
// cudaGetSymbolAddress, with that device current, and that address is what the kernels receive.
//
// Limits and rules
//   * M * A * N <= kNoAllocFloats (4 Mi floats = 16 MiB; e.g. 100 tokens x 10 slots x 4096 columns).  Larger calls are
//     refused with an error; use the caller-scratch entry point for them.
//   * The 16 MiB are taken on a device when the CUDA runtime loads this part of the library there, and held until the
//     process exits.  With the runtime's default lazy loading that moment is the FIRST CALL of this entry point on the
//     device (which also loads the combine's kernels): a host that plans its device memory to the last byte makes one
//     small call per device BEFORE it sizes that plan, or the first call of a decode step can fail for lack of memory.
//   * That first call also performs the address lookup (a blocking runtime call): make it before any stream capture.
//   * The looked-up address is kept per device ordinal for the life of the process; cudaDeviceReset, or driving the
//     same device through another context, invalidates it.
//   * All calls on a device share the one array and it keeps the last call's contents.  Nothing in it needs to start
//     at zero - every word a call reads was written by that same call - but two calls that overlap on the GPU (two
//     streams, or two host threads) race on it.  Serialize them.
//   * Nothing here calls cudaMalloc, cudaFree or an allocating library routine.

#include "experts.cuh"

#include <mutex>

namespace sxb {
namespace {

constexpr int64_t kNoAllocFloats = 4ll << 20;  // 16 MiB of FP32 per-slot dots

static __device__ __align__(256) float g_partial[kNoAllocFloats];

// The array's device address on the current device, looked up on first use (one slot per device ordinal).
int partial_scratch(float **out) {
    static std::mutex mu;
    static float *addr[64] = {};
    int dev = -1;
    SXB_CUDA(cudaGetDevice(&dev), "combine_grouped_noalloc: no current device");
    SXB_CHECK(dev >= 0 && dev < 64, "combine_grouped_noalloc: device ordinal ", dev, " outside 0..63");
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void *p = nullptr;
        SXB_CUDA(cudaGetSymbolAddress(&p, g_partial), "combine_grouped_noalloc: looking up the scratch array on device ", dev);
        SXB_CHECK(p != nullptr, "combine_grouped_noalloc: the scratch array has no address on device ", dev);
        addr[dev] = static_cast<float *>(p);
    }
    *out = addr[dev];
    return SXB_OK;
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" int sxb_linear_q4_experts_combine_grouped_noalloc(const void *h, const SxbQView *w, int64_t E, const int32_t *ids,
                                                             const float *coef, const void *ws, size_t ws_bytes, int64_t M,
                                                             int64_t A, void *y, int act, int out_act, int math,
                                                             sxb_stream_t stream, const SxbMoeSharedAdd *shared, int h_f16) {
    const char *fn = "linear_q4_experts_combine_grouped_noalloc";
    SXB_CHECK(w != nullptr && E >= 1 && w->N >= 1 && w->N % E == 0, fn, ": weight has ", w ? w->N : 0, " rows for E = ", E, " experts");
    SXB_CHECK(M >= 1 && A >= 1, fn, ": M = ", M, ", A = ", A, ", both must be >= 1");
    const int64_t N = w->N / E;
    SXB_CHECK(M * A <= kNoAllocFloats / N, fn, ": M * A * N = ", M, " * ", A, " * ", N, " per-slot dots exceed the built-in scratch of ",
              kNoAllocFloats, " floats (16 MiB); call linear_q4_experts_combine_grouped with caller-owned scratch instead");
    float *partial = nullptr;
    if (int rc = partial_scratch(&partial)) return rc;
    // from here on the caller-scratch entry point's own code: the same checks (pointers, dtypes, overlaps), the same kernels
    return combine_grouped<4>(fn, h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, out_act, math, stream, shared, h_f16, E, 0);
}
