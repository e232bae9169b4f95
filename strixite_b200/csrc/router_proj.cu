// The router-logits projection, the step right before the MoE router: logits [M, N] = x [M, K] * W^T (+ bias), FP32 out
// (runtime/qwen4exp.cpp:3149-3155; kernels/linear.hip:82-132 linear_bf16w, kernels/linear_wmma.hip:115-151
// linear_bf16w_wmma), and the residual add that closes a sublayer.
//
// Two forms, by regime:
//   * streaming (decode, a few dozen tokens): a warp owns one weight row and streams it once for all tokens; the row's
//     bytes (FP32 or BF16) come by 16-byte loads, the tokens' activations from L2.  HBM-bound on the weight;
//   * tcgen05 (prefill, thousands of tokens): a plain tensor-core GEMM with both operands staged by tensor copies.  The
//     weight is the reference's BF16 [N, K], or an FP32 one split once, at load time, into P BF16 "planes"
//     W = W1 + W2 (+ W3) (each plane the BF16 rounding of what the planes before it left over), so that the products
//     x * Wp are exact BF16 x BF16 products and their FP32 sum carries 16 (P = 2) or 24 (P = 3) bits of the weight.
//     The weight rows sit on the MMA's M (128 a tile), the tokens on its N (128), accumulators double-buffered in
//     tensor memory; warp 0 issues the copies, warp 1 the MMAs, warps 2-5 are the epilogue (bias add, FP32 store,
//     a token's 32 experts of a warp are 128 contiguous bytes).
// Every device-side wait is bounded; one that runs out is recorded in the library's status words (see
// sxb_check_dense_status) and the kernel returns.

#include "experts.cuh"
#include "tc_ptx.cuh"

#include <algorithm>

namespace sxb {
namespace {

// ---- streaming form ------------------------------------------------------------------------------------------

constexpr int kStreamRows = 8;    // weight rows a CTA takes at a time
constexpr int kStreamWarps = 2 * kStreamRows;  // two warps per row, each streaming half of the staged k range
constexpr int kTokChunk = 16;     // tokens whose activations sit in shared memory (and whose sums a lane keeps)
constexpr int kStreamKTile = 4096;  // k range staged at a time: 16 tokens x 4096 x 2 bytes = 128 KB of shared memory
constexpr int kRunsPerLane = kStreamKTile / 2 / 8 / 32;  // runs of eight k a lane takes from its half of a full tile: 8

__device__ inline void load_w8(const float *p, float (&w)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    w[0] = a.x, w[1] = a.y, w[2] = a.z, w[3] = a.w, w[4] = b.x, w[5] = b.y, w[6] = b.z, w[7] = b.w;
}
__device__ inline void load_w8(const uint16_t *p, float (&w)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) w[2 * i] = __uint_as_float(u[i] << 16), w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
}

// y[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]).  A CTA stages the activations of 16 tokens in shared memory once and
// streams eight weight rows against them, two warps a row (one per half of the staged k range).  A lane issues ALL the
// loads of its part of the row before it consumes any of them - with a few dozen tokens the kernel is one memory round
// trip plus arithmetic, so what counts is how many bytes are in flight.  The sum of a (token, row) pair is formed in a
// fixed order: per lane ascending k, an xor butterfly in the warp, then the row's two halves in order.
template <typename TW, typename TOUT>
__global__ void __launch_bounds__(32 * kStreamWarps)
    logits_stream_kernel(const uint16_t *__restrict__ x, const TW *__restrict__ w, const float *__restrict__ bias, int64_t M,
                         int64_t N, int64_t K, TOUT *__restrict__ y, int64_t ld) {
    extern __shared__ __align__(16) unsigned char xs_raw[];
    uint4 *xs = reinterpret_cast<uint4 *>(xs_raw);  // [kTokChunk][kt / 8] chunks of eight BF16
    __shared__ float part[kStreamWarps][kTokChunk];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, half = warp & 1;
    const int64_t n = (int64_t)blockIdx.x * kStreamRows + (warp >> 1);
    const bool row_ok = n < N;
    const TW *wr = w + (row_ok ? n : 0) * K;
    const float b = (row_ok && bias) ? bias[n] : 0.f;
    for (int64_t m0 = 0; m0 < M; m0 += kTokChunk) {
        const int live = (int)min((int64_t)kTokChunk, M - m0);
        float acc[kTokChunk];
#pragma unroll
        for (int t = 0; t < kTokChunk; ++t) acc[t] = 0.f;
        for (int64_t k0 = 0; k0 < K; k0 += kStreamKTile) {
            const int kt = (int)min((int64_t)kStreamKTile, K - k0), chunks = kt / 8;
            // this warp's half of the tile, in runs of eight k: [c_lo, c_hi)
            const int c_lo = half * ((chunks + 1) / 2), c_hi = half ? chunks : (chunks + 1) / 2;
            float wv[kRunsPerLane][8];
#pragma unroll
            for (int j = 0; j < kRunsPerLane; ++j) {  // the row's bytes first: they come from HBM
                const int c = c_lo + lane + 32 * j;
                if (row_ok && c < c_hi) load_w8(wr + k0 + (int64_t)c * 8, wv[j]);
            }
            __syncthreads();  // every warp is done with the previous tile
            for (int i = threadIdx.x; i < kTokChunk * chunks; i += 32 * kStreamWarps) {
                const int t = i / chunks, c = i % chunks;
                xs[i] = t < live ? __ldg(reinterpret_cast<const uint4 *>(x + (m0 + t) * K + k0) + c) : make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();
            if (row_ok) {
#pragma unroll
                for (int j = 0; j < kRunsPerLane; ++j) {
                    const int c = c_lo + lane + 32 * j;
                    if (c >= c_hi) break;
#pragma unroll
                    for (int t = 0; t < kTokChunk; ++t) {
                        const uint4 xv = xs[t * chunks + c];
                        const uint32_t u[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            acc[t] = fmaf(__uint_as_float(u[i] << 16), wv[j][2 * i], acc[t]);
                            acc[t] = fmaf(__uint_as_float(u[i] & 0xffff0000u), wv[j][2 * i + 1], acc[t]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kTokChunk; ++t) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], off);
            if (lane == 0) part[warp][t] = acc[t];
        }
        __syncthreads();
        if (half == 0 && lane < live && row_ok) store_from_f32(y, (m0 + lane) * ld + n, part[warp][lane] + part[warp + 1][lane] + b);
        __syncthreads();
    }
}

// x_out = bf16(x + y): the residual add that closes the sublayer (the reference injects into its four residual streams
// with hc_inject, kernels/hc.hpp:52-54; this is the single-stream case with weight 1).  Eight elements a thread.
template <typename TY>
__global__ void __launch_bounds__(256) residual_add_kernel(const uint4 *__restrict__ x, const TY *__restrict__ y, uint4 *__restrict__ out,
                                                           int64_t chunks) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 xv = x[i];
        const uint32_t u[4] = {xv.x, xv.y, xv.z, xv.w};
        float yv[8];
        if constexpr (sizeof(TY) == 4) {
            const float4 a = reinterpret_cast<const float4 *>(y)[2 * i], b = reinterpret_cast<const float4 *>(y)[2 * i + 1];
            yv[0] = a.x, yv[1] = a.y, yv[2] = a.z, yv[3] = a.w, yv[4] = b.x, yv[5] = b.y, yv[6] = b.z, yv[7] = b.w;
        } else {
            const uint4 a = reinterpret_cast<const uint4 *>(y)[i];
            const uint32_t v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) yv[2 * j] = __uint_as_float(v[j] << 16), yv[2 * j + 1] = __uint_as_float(v[j] & 0xffff0000u);
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = f32_to_bf16_bits(__uint_as_float(u[j] << 16) + yv[2 * j]);
            const uint32_t hi = f32_to_bf16_bits(__uint_as_float(u[j] & 0xffff0000u) + yv[2 * j + 1]);
            o[j] = lo | (hi << 16);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- tcgen05 form ----------------------------------------------------------------------------------------------

constexpr int kGemmThreads = 192;      // warp 0 copies, warp 1 MMA issue, warps 2-5 epilogue
constexpr int kTile = 128;             // weight rows (MMA M) and tokens (MMA N) of a tile
constexpr int kGemmBK = 64;            // k per stage: one 128-byte swizzle line of BF16
constexpr int kOperandBytes = kTile * kGemmBK * 2;  // 16 KB: one operand tile of one k-block
constexpr int kMaxStages = 4;
constexpr int kMaxPlanes = 3;
constexpr int kGemmTmemCols = 256;     // two accumulators of 128 token columns

struct GemmArgs {
    const float *bias;
    float *logits;
    int64_t M, N, Npad, K, ld;
    int planes, stages;
    uint32_t *status;
    unsigned long long wait_limit_ns;
};

// Instruction descriptor for kind::f16 with BF16 operands: D FP32 (bits [4,6) = 1), A and B BF16 (bits [7,10) and
// [10,13) = 1), both K-major, N >> 3 at bits [17,23), M >> 4 at bits [24,29).
__device__ inline uint32_t instr_desc_bf16(int n_cols) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n_cols >> 3) << 17) | ((128u >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem].  Whole-warp call, one elected lane issues (as tc_commit).
__device__ inline void tc_mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ inline void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__global__ void __launch_bounds__(kGemmThreads, 1)
    logits_gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full[2], acc_empty[2], drain_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (int)(a.K / kGemmBK), n_rb = (int)(a.Npad / kTile), n_tt = (int)((a.M + kTile - 1) / kTile);
    const int n_items = n_rb * n_tt;
    const int stage_bytes = (1 + a.planes) * kOperandBytes;
    volatile int *abort_v = &abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) mbar_init(&full_bar[s], 1), mbar_init(&empty_bar[s], 1);
        for (int b = 0; b < 2; ++b) mbar_init(&acc_full[b], 1), mbar_init(&acc_empty[b], 4);
        mbar_init(&drain_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_smem)), "r"(kGemmTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    auto raise_abort = [&](int item, int role) {
        if (atomicExch(&abort_flag, 1) == 0 && atomicCAS(&a.status[0], 0u, 2u) == 0u) {
            a.status[1] = (uint32_t)item;
            a.status[2] = (uint32_t)role;
        }
    };

    uint32_t issued = 0;  // stages filled by this thread (the copy thread only)
    if (warp == 0) {
        // ===================== copies: one thread, as far ahead as free stages allow =====================
        if (lane == 0) {
            for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
                const int tile = item / n_rb, rb = item % n_rb;
                for (int kb = 0; kb < n_kb; ++kb, ++issued) {
                    const int stage = issued % a.stages;
                    if (issued >= (uint32_t)a.stages &&
                        !mbar_wait(&empty_bar[stage], ((issued / a.stages) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) {
                        raise_abort(item, 5);
                        break;
                    }
                    const uint32_t dst = smem_u32(smem + stage * stage_bytes);
                    mbar_expect_tx(&full_bar[stage], (uint32_t)stage_bytes);
                    tma_load_2d(dst, &xmap, kb * kGemmBK, tile * kTile, &full_bar[stage]);
                    for (int p = 0; p < a.planes; ++p)
                        tma_load_2d(dst + (1 + p) * kOperandBytes, &wmap, kb * kGemmBK, (int)(p * a.Npad) + rb * kTile, &full_bar[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issue =====================
        uint32_t count = 0, acc_count = 0;
        const uint32_t idesc = instr_desc_bf16(kTile);
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x, ++acc_count) {
            const uint32_t buf = acc_count & 1u;
            if (lane == 0 && acc_count >= 2 && !mbar_wait(&acc_empty[buf], ((acc_count >> 1) & 1u) ^ 1u, abort_v, a.wait_limit_ns))
                raise_abort(item, 2);
            __syncwarp();
            if (*abort_v) break;
            tc_fence_after();
            const uint32_t d = tmem_base + buf * (uint32_t)kTile;
            bool failed = false;
            for (int kb = 0; kb < n_kb; ++kb, ++count) {
                const int stage = count % a.stages;
                if (lane == 0 && !mbar_wait(&full_bar[stage], (count / a.stages) & 1u, abort_v, a.wait_limit_ns))
                    raise_abort(item, 3), failed = true;
                if (__any_sync(0xffffffffu, failed)) break;
                tc_fence_after();
                const uint32_t base = smem_u32(smem + stage * stage_bytes);
                const uint64_t b_desc = smem_desc(base);
                for (int p = 0; p < a.planes; ++p) {
                    const uint64_t a_desc = smem_desc(base + (uint32_t)((1 + p) * kOperandBytes));
#pragma unroll
                    for (int j = 0; j < kGemmBK / 16; ++j)  // k = 16 an instruction: 32 bytes further along the swizzled line
                        tc_mma_f16_ss(d, a_desc + 2 * j, b_desc + 2 * j, idesc, (kb | p | j) != 0);
                }
                tc_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
            }
            if (__any_sync(0xffffffffu, failed)) break;
            tc_commit(&acc_full[buf]);
        }
        // every MMA of this CTA has completed before tensor memory is released (not given up while aborting)
        tc_commit(&drain_bar);
        if (lane == 0) mbar_wait(&drain_bar, 0u, nullptr, a.wait_limit_ns);
        __syncwarp();
    } else {
        // ===================== epilogue =====================
        const int quad = warp & 3;  // the tensor-memory lanes a warp may read: 32 (warp % 4) ..
        uint32_t acc_count = 0;
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x, ++acc_count) {
            const int tile = item / n_rb, rb = item % n_rb;
            const uint32_t buf = acc_count & 1u;
            if (lane == 0 && !mbar_wait(&acc_full[buf], (acc_count >> 1) & 1u, abort_v, a.wait_limit_ns)) raise_abort(item, 4);
            __syncwarp();
            if (*abort_v) break;
            tc_fence_after();
            const int64_t e = (int64_t)rb * kTile + quad * 32 + lane;
            const bool row_ok = e < a.N;
            const float b = (row_ok && a.bias) ? a.bias[e] : 0.f;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * (uint32_t)kTile;
            const int64_t t0 = (int64_t)tile * kTile;
            for (int c0 = 0; c0 < kTile; c0 += 16) {
                float v[16];
                tc_ld16(taddr + (uint32_t)c0, v);
                if (c0 + 16 == kTile) {  // the last columns are in registers: the accumulator may be overwritten
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                }
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    const int64_t tok = t0 + c0 + t;
                    if (row_ok && tok < a.M) a.logits[tok * a.ld + e] = v[t] + b;
                }
            }
        }
    }

    // an aborting CTA waits (bounded) for the copies it issued before its shared memory can go to another CTA
    if (*abort_v && issued > 0)
        for (int s = 0; s < a.stages; ++s) {
            if (issued <= (uint32_t)s) continue;
            const uint32_t last = ((issued - 1 - (uint32_t)s) / a.stages) * a.stages + (uint32_t)s;
            mbar_wait(&full_bar[s], (last / a.stages) & 1u, nullptr, 1000000ull);
        }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kGemmTmemCols) : "memory");
    }
}

// W [N, K] (FP32 or BF16) -> P BF16 planes [P][Npad][K]: plane p holds the BF16 rounding of what the planes before it left
// of the weight; rows N .. Npad - 1 are zero.  With a BF16 weight one plane is the weight itself.
template <typename TW>
__global__ void __launch_bounds__(256) split_planes_kernel(const TW *__restrict__ w, int64_t N, int64_t Npad, int64_t K, int planes,
                                                           uint16_t *__restrict__ out) {
    const int64_t total = Npad * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float r = i / K < N ? load_as_f32(w, i) : 0.f;
        for (int p = 0; p < planes; ++p) {
            const uint16_t b = f32_to_bf16_bits(r);
            out[(int64_t)p * total + i] = b;
            r -= bf16_bits_to_f32(b);  // exact: the difference of an FP32 value and its BF16 rounding fits FP32
        }
    }
}

int64_t pad_rows(int64_t N) { return (N + kTile - 1) / kTile * kTile; }

int check_proj(const char *fn, const void *x, const void *w, const void *y, int64_t M, int64_t N, int64_t K) {
    SXB_CHECK(x != nullptr && w != nullptr && y != nullptr, fn, ": null pointer (x=", x, ", w=", w, ", y=", y, ")");
    SXB_CHECK(M >= 1 && N >= 1 && N <= (1 << 24) && K >= 8 && K % 8 == 0 && K <= (1 << 24), fn, ": M = ", M, ", N = ", N, ", K = ", K,
              " (K a multiple of 8)");
    SXB_CHECK(aligned16(x) && aligned16(w), fn, ": x and w must be 16-byte aligned");
    return SXB_OK;
}

template <typename TOUT>
int launch_stream_logits(const char *fn, const void *x, const void *w, int w_act, const float *bias, int64_t M, int64_t N, int64_t K,
                         TOUT *y, int64_t ld, cudaStream_t st) {
    const unsigned blocks = (unsigned)((N + kStreamRows - 1) / kStreamRows);
    const size_t smem = (size_t)kTokChunk * std::min<int64_t>(K, kStreamKTile) * 2;
    if (w_act == SXB_ACT_F32) {
        auto kern = logits_stream_kernel<float, TOUT>;
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory");
        kern<<<blocks, 32 * kStreamWarps, smem, st>>>((const uint16_t *)x, (const float *)w, bias, M, N, K, y, ld);
    } else {
        auto kern = logits_stream_kernel<uint16_t, TOUT>;
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory");
        kern<<<blocks, 32 * kStreamWarps, smem, st>>>((const uint16_t *)x, (const uint16_t *)w, bias, M, N, K, y, ld);
    }
    SXB_CHECK_LAUNCH(fn, " M=", M, " N=", N, " K=", K);
    return SXB_OK;
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" {

int sxb_linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, int act, int out_act,
                     sxb_stream_t stream) {
    const char *fn = "linear_bf16w";
    if (int rc = check_proj(fn, x, w, y, M, N, K)) return rc;
    SXB_CHECK(act == SXB_ACT_BF16, fn, ": BF16 activations only, got ", act);
    SXB_CHECK(out_act == SXB_ACT_BF16 || out_act == SXB_ACT_F32, fn, ": output dtype ", out_act, " unsupported (BF16, or F32)");
    SXB_CHECK(apart(x, M * K * 2, y, M * N * act_bytes(out_act)), fn, ": y overlaps x");
    auto st = static_cast<cudaStream_t>(stream);
    return out_act == SXB_ACT_F32 ? launch_stream_logits<float>(fn, x, w, SXB_ACT_BF16, nullptr, M, N, K, (float *)y, N, st)
                                  : launch_stream_logits<uint16_t>(fn, x, w, SXB_ACT_BF16, nullptr, M, N, K, (uint16_t *)y, N, st);
}

int sxb_router_logits(const void *x, const void *w, int w_act, const float *bias, int64_t M, int64_t N, int64_t K, float *logits,
                      int64_t ld, sxb_stream_t stream) {
    const char *fn = "router_logits";
    if (int rc = check_proj(fn, x, w, logits, M, N, K)) return rc;
    SXB_CHECK(w_act == SXB_ACT_F32 || w_act == SXB_ACT_BF16, fn, ": weight dtype ", w_act, " unsupported (F32 or BF16)");
    SXB_CHECK(ld >= N, fn, ": logits row stride ld = ", ld, " < N = ", N);
    SXB_CHECK(apart(x, M * K * 2, logits, M * ld * 4), fn, ": logits overlap x");
    return launch_stream_logits<float>(fn, x, w, w_act, bias, M, N, K, logits, ld, static_cast<cudaStream_t>(stream));
}

size_t sxb_router_planes_bytes(int64_t N, int64_t K, int planes) {
    if (!(N >= 1 && K >= 1 && planes >= 1 && planes <= kMaxPlanes)) {
        fail_check(SXB_FILE_, __LINE__, __func__, "N >= 1 && K >= 1 && 1 <= planes <= 3",
                   cat("router_planes_bytes: N = ", N, ", K = ", K, ", planes = ", planes));
        return 0;
    }
    return (size_t)planes * (size_t)pad_rows(N) * (size_t)K * 2;
}

int sxb_router_prepare(const void *w, int w_act, int64_t N, int64_t K, int planes, void *planes_out, sxb_stream_t stream) {
    const char *fn = "router_prepare";
    SXB_CHECK(w != nullptr && planes_out != nullptr, fn, ": null pointer");
    SXB_CHECK(w_act == SXB_ACT_F32 || w_act == SXB_ACT_BF16, fn, ": weight dtype ", w_act, " unsupported (F32 or BF16)");
    SXB_CHECK(planes >= 1 && planes <= kMaxPlanes, fn, ": planes = ", planes, ", expected 1..", kMaxPlanes);
    SXB_CHECK(N >= 1 && K >= 64 && K % 64 == 0 && K <= (1 << 24), fn, ": N = ", N, ", K = ", K, " (K a multiple of 64)");
    SXB_CHECK(aligned16(planes_out), fn, ": the planes must be 16-byte aligned");
    const int64_t Npad = pad_rows(N);
    const unsigned blocks = (unsigned)std::min<int64_t>((Npad * K + 255) / 256, (int64_t)sm_count() * 8);
    auto st = static_cast<cudaStream_t>(stream);
    if (w_act == SXB_ACT_F32) split_planes_kernel<float><<<blocks, 256, 0, st>>>((const float *)w, N, Npad, K, planes, (uint16_t *)planes_out);
    else split_planes_kernel<uint16_t><<<blocks, 256, 0, st>>>((const uint16_t *)w, N, Npad, K, planes, (uint16_t *)planes_out);
    SXB_CHECK_LAUNCH(fn, " N=", N, " K=", K, " planes=", planes);
    return SXB_OK;
}

int sxb_router_logits_wmma(const void *x, const void *planes_in, int planes, const float *bias, int64_t M, int64_t N, int64_t K,
                           float *logits, int64_t ld, sxb_stream_t stream) {
    const char *fn = "router_logits_wmma";
    if (int rc = check_proj(fn, x, planes_in, logits, M, N, K)) return rc;
    SXB_CHECK(planes >= 1 && planes <= kMaxPlanes, fn, ": planes = ", planes, ", expected 1..", kMaxPlanes);
    SXB_CHECK(K % kGemmBK == 0, fn, ": K = ", K, " must be a multiple of ", kGemmBK);
    SXB_CHECK(M <= (1 << 24), fn, ": M = ", M, " tokens, expected <= 2^24");
    SXB_CHECK(ld >= N, fn, ": logits row stride ld = ", ld, " < N = ", N);
    SXB_CHECK(apart(x, M * K * 2, logits, M * ld * 4), fn, ": logits overlap x");
    GemmArgs a{};
    a.bias = bias, a.logits = logits, a.M = M, a.N = N, a.Npad = pad_rows(N), a.K = K, a.ld = ld, a.planes = planes;
    a.stages = planes == 3 ? 3 : 4;
    a.wait_limit_ns = wait_limit_ns();
    if (int rc = library_status_words(fn, &a.status)) return rc;
    CUtensorMap xmap, wmap;
    if (int rc = tensor_map_2d(fn, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kGemmBK, kTile,
                               CU_TENSOR_MAP_SWIZZLE_128B, &xmap))
        return rc;
    // one plane may be the raw BF16 weight [N, K] itself: its rows past N read as zero instead of being stored as zeros
    if (int rc = tensor_map_2d(fn, planes_in, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)(planes == 1 ? N : planes * a.Npad), (uint64_t)K * 2,
                               kGemmBK, kTile, CU_TENSOR_MAP_SWIZZLE_128B, &wmap))
        return rc;
    const size_t smem = (size_t)a.stages * (1 + planes) * kOperandBytes + 1024;
    SXB_CUDA(cudaFuncSetAttribute(logits_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory");
    const int64_t items = (a.Npad / kTile) * ((M + kTile - 1) / kTile);
    const unsigned grid = (unsigned)std::min<int64_t>(items, sm_count());
    logits_gemm_kernel<<<grid, kGemmThreads, smem, static_cast<cudaStream_t>(stream)>>>(a, xmap, wmap);
    SXB_CHECK_LAUNCH(fn, " M=", M, " N=", N, " K=", K, " planes=", planes);
    return SXB_OK;
}

int sxb_residual_add(const void *x, const void *y, int y_act, void *out, int64_t n, sxb_stream_t stream) {
    const char *fn = "residual_add";
    SXB_CHECK(x != nullptr && y != nullptr && out != nullptr, fn, ": null pointer");
    SXB_CHECK(n >= 8 && n % 8 == 0, fn, ": n = ", n, " elements, expected a positive multiple of 8");
    SXB_CHECK(y_act == SXB_ACT_F32 || y_act == SXB_ACT_BF16, fn, ": dtype of y ", y_act, " unsupported (F32 or BF16)");
    SXB_CHECK(aligned16(x) && aligned16(y) && aligned16(out), fn, ": x, y and out must be 16-byte aligned");
    SXB_CHECK(apart(out, n * 2, y, n * act_bytes(y_act)), fn, ": out overlaps y");
    const int64_t chunks = n / 8;
    const unsigned blocks = (unsigned)std::min<int64_t>((chunks + 255) / 256, (int64_t)sm_count() * 8);
    auto st = static_cast<cudaStream_t>(stream);
    if (y_act == SXB_ACT_F32) residual_add_kernel<float><<<blocks, 256, 0, st>>>((const uint4 *)x, (const float *)y, (uint4 *)out, chunks);
    else residual_add_kernel<uint16_t><<<blocks, 256, 0, st>>>((const uint4 *)x, (const uint16_t *)y, (uint4 *)out, chunks);
    SXB_CHECK_LAUNCH(fn, " n=", n);
    return SXB_OK;
}

}  // extern "C"
