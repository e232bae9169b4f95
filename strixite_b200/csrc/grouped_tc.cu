// Grouped expert GEMMs for the dense-contraction regime (prefill: thousands of tokens, ~80 and up per expert) on the
// 5th-generation tensor cores: tcgen05.mma with FP32 accumulators in tensor memory.  C ABI side: the MoeMath::WmmaF16
// forms of linear_q*_experts_gather_grouped[_swiglu] / _combine_grouped (kernels/moe_grouped.hpp:58-91).
//
// Numerics are those of the reference's matrix-unit path (kernels/moe_grouped.hpp:29-38, kernels/wmma_gemm.hpp:116-129):
// activations as F16 (exact from BF16 in F16's range), weights dequantized to F16 as code * scale + min with one
// rounding, FP32 accumulation over the whole K, and - fused SwiGLU - h = silu(g) * u from the FP32 accumulators,
// rounded once to BF16 (kernels/moe_grouped.hip:508-524).
//
// Shape of the computation ("swap AB"): the weight rows sit on the MMA's M (128 per instruction, two accumulators =
// 256 rows per work item) and the tokens of one expert on its N (a multiple of 16 up to 128), so an expert with 80
// tokens costs 80 columns, not a padded 128-row tile.  D[row, token] lives in tensor memory, one row per TMEM lane:
// the epilogue thread of lane j holds gate row j and up row j of the same tokens, and SwiGLU needs no data movement.
//
// One persistent CTA per SM, warp-specialised:
//   warps 0-3   epilogue: tcgen05.ld of a finished accumulator pair -> SwiGLU / stores, while the next item runs
//   warp  4     one elected thread issues tcgen05.mma (operands: shared-memory descriptors, K-major, 128-byte swizzle)
//   warps 5-12  producers.  Thread p owns weight row p of the item: it streams the row's packed codes from global
//               memory 128 bytes at a time (kept in registers one super-block ahead), dequantizes 64 codes per k-block
//               with lop3 / packed-half arithmetic and writes the row's 128-byte line of the A tile.  The same
//               threads gather the tokens' activation rows (16 bytes a chunk), convert BF16 -> F16 and write the B
//               tile.  Within every group of 8 consecutive k both operands use the order [0 4 1 5 2 6 3 7] (Q4),
//               the order in which a nibble pair falls out of one lop3, so no element is moved after dequantization.
// Stages are handed over with mbarriers (producers -> MMA: arrive after fence.proxy.async; MMA -> producers and
// MMA -> epilogue: tcgen05.commit).  Every wait is bounded: past the limit the CTA raises its abort flag, records
// {2, item, role} in the status words, drains the tensor pipe and frees its tensor memory before returning.
//
// No tensor map, no multicast: the operands never come through TMA, so nothing here can touch a peer GPU's memory.

#include "experts.cuh"

#include <cuda_fp16.h>

#ifdef SXB_TC_PROF
__device__ unsigned long long g_tc_prof[32];
__device__ long long g_tc_trace[4][64][2];  // role (A, B, MMA, -), k-block index of CTA 0, two timestamps
#define TRACE(role, idx, which) \
    do { if (blockIdx.x == 0 && lane == 0 && (idx) < 64) g_tc_trace[role][idx][which] = clock64(); } while (0)
#else
#define TRACE(role, idx, which) do {} while (0)
#endif

namespace sxb {
namespace {

// warps 0-3 epilogue, 4-5 MMA issue (one per accumulator), 6-13 weight producers, 14-15 activation producers
constexpr int kEpiWarps = 4, kMmaWarp = 4, kMmaWarps = 2, kFirstAWarp = kMmaWarp + kMmaWarps, kAWarps = 8,
              kFirstBWarp = kFirstAWarp + kAWarps, kBWarps = 2;
constexpr int kThreads = 32 * (kFirstBWarp + kBWarps);  // 512
constexpr int kAThreads = 32 * kAWarps;                 // 256 = weight rows per item
constexpr int kProducers = kAThreads;
constexpr int kBPrefetch = 12;                          // k-blocks of tile-blocked activations pulled into L2 ahead of their copy
constexpr int kBAhead = 2;                              // k-blocks of activations in flight (cp.async groups)
constexpr int kBK = 64;                                               // k per stage: one 128-byte swizzle line of F16
constexpr int kMaxTileTokens = 128;
constexpr int kStages = 4;
constexpr int kBBytes = kMaxTileTokens * kBK * 2;   // 16 KB: the activation tile of one k-block
constexpr int kStageBytes = kBBytes;                // shared memory per stage (the weights travel through tensor memory)
// Tensor memory, 512 columns x 128 lanes: two accumulators (weight rows 0-127 and 128-255 of the item) of up to 128 token
// columns each, then kStages stages of the A operand - per stage and accumulator 32 columns = 64 F16 of one weight row
// per lane.
constexpr int kTmemCols = 512;
constexpr int kAccCols = kMaxTileTokens;
constexpr int kAStageCol0 = 2 * kAccCols, kAStageCols = 2 * (kBK / 2);
// Epilogue staging in shared memory: FP32 [accumulator][token][row], token stride padded to 132 words so that the drain
// (lane = row) and the read-back (8 consecutive rows of a token per thread) are both free of bank conflicts.
constexpr int kEpiTokStride = 132;
constexpr int kEpiBytes = 2 * kMaxTileTokens * kEpiTokStride * 4;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s: far beyond any legitimate wait

enum TcMode { kTcGather = 0, kTcSwiglu = 1, kTcPartial = 2 };

// Optional cycle accounting per warp role (development builds only: -DSXB_TC_PROF).  CTA 0, lane 0 of one warp per role.
#ifdef SXB_TC_PROF
#define PROF_BEGIN() const long long prof_t0_ = clock64()
#define PROF_ADD(slot) \
    do { if (blockIdx.x == 0 && lane == 0) atomicAdd(&g_tc_prof[slot], (unsigned long long)(clock64() - prof_t0_)); } while (0)
#define PROF_COUNT(slot) \
    do { if (blockIdx.x == 0 && lane == 0) atomicAdd(&g_tc_prof[slot], 1ull); } while (0)
#else
#define PROF_BEGIN() do {} while (0)
#define PROF_ADD(slot) do {} while (0)
#define PROF_COUNT(slot) do {} while (0)
#endif

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
};

// ---- PTX wrappers ----------------------------------------------------------------------------------------------
__device__ inline uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ inline void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ inline void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
#ifdef SXB_TC_EXP_TESTWAIT
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ inline unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  False when the CTA is aborting or the limit ran out (then the caller raises the abort itself).
// The common case must stay cheap: the first polls touch nothing but the barrier; the abort flag and the (slow to read)
// global timer are consulted only once a wait has lasted thousands of polls.
__device__ inline bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t spins = 0;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 4095u) == 4095u) {
            if (*abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) return false;
        }
    }
}
__device__ inline void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive columns of this thread's TMEM lane.
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

// 16 consecutive columns of this thread's TMEM lane, written from registers.
__device__ inline void tc_st16(uint32_t taddr, const uint4 (&d)[4]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(d[0].x), "r"(d[0].y), "r"(d[0].z), "r"(d[0].w), "r"(d[1].x), "r"(d[1].y), "r"(d[1].z), "r"(d[1].w), "r"(d[2].x),
        "r"(d[2].y), "r"(d[2].z), "r"(d[2].w), "r"(d[3].x), "r"(d[3].y), "r"(d[3].z), "r"(d[3].w)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 k of F16, two per 32-bit column) read from tensor memory.
__device__ inline void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
//   bits [0,14) start address >> 4 | [16,30) leading byte offset >> 4 (unused for swizzled K-major: 1)
//   [32,46) stride byte offset >> 4 (1024 B) | [46,48) descriptor version 1 | [61,64) layout 2 = SWIZZLE_128B
__device__ inline uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: D FP32 (bits [4,6) = 1), A and B F16 (formats 0), both K-major,
// N >> 3 at bits [17,23), M >> 4 at bits [24,29).
__device__ inline uint32_t instr_desc(int n_cols) { return (1u << 4) | ((uint32_t)(n_cols >> 3) << 17) | ((128u >> 4) << 24); }

__device__ inline uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ inline __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

// Byte offset of 16-byte chunk c of row r inside a K-major, 128-byte-swizzled tile.
__device__ inline uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// Tile-blocked activations: rows live at their position `pos` in the pack's slot order, k-block-major, each row's 128-byte
// line of a k-block already swizzled for its place n = pos - tile_start in the tile.  The B operand of (tile, k-block) is
// then ONE contiguous run of cnt * 128 bytes at byte offset (kb * S + tile_start) * 128: a single bulk copy.
__device__ inline int64_t tiled_offset(int64_t S, int kb, int64_t pos, int n, int c) {
    return ((int64_t)kb * S + pos) * 128 + ((c ^ (n & 7)) << 4);
}
__device__ inline void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ inline void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Eight activations (one 16-byte chunk of BF16 or F16) -> F16 in the operand's k order.
template <int BITS>
__device__ inline uint4 b_chunk(uint4 s, bool is_f16) {
    uint4 d;
    if (is_f16) {
        if (BITS == 4) {
            d.x = __byte_perm(s.x, s.z, 0x5410), d.y = __byte_perm(s.x, s.z, 0x7632);
            d.z = __byte_perm(s.y, s.w, 0x5410), d.w = __byte_perm(s.y, s.w, 0x7632);
        } else {
            d = s;
        }
        return d;
    }
    const uint32_t w[4] = {s.x, s.y, s.z, s.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[2 * i] = __uint_as_float(w[i] << 16), f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    if (BITS == 4) {  // [x0 x4 | x1 x5 | x2 x6 | x3 x7]
        d.x = h2_as_u32(__floats2half2_rn(f[0], f[4])), d.y = h2_as_u32(__floats2half2_rn(f[1], f[5]));
        d.z = h2_as_u32(__floats2half2_rn(f[2], f[6])), d.w = h2_as_u32(__floats2half2_rn(f[3], f[7]));
    } else {
        d.x = h2_as_u32(__floats2half2_rn(f[0], f[1])), d.y = h2_as_u32(__floats2half2_rn(f[2], f[3]));
        d.z = h2_as_u32(__floats2half2_rn(f[4], f[5])), d.w = h2_as_u32(__floats2half2_rn(f[6], f[7]));
    }
    return d;
}

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

struct ItemInfo {
    int bucket, start, cnt;  // expert (bucket E = invalid ids), first position in slots[], tokens in the tile
    int rb;                  // row block
};

template <int MODE>
__device__ inline int row_blocks(const TcArgs &a) {
    return MODE == kTcSwiglu ? (int)((a.N / 2 + 127) / 128) : (int)((a.N + kProducers - 1) / kProducers);
}
template <int MODE>
__device__ inline ItemInfo item_info(const TcArgs &a, int item, int rbs) {
    ItemInfo it;
    const int tile = item / rbs;
    it.rb = item % rbs;
    it.bucket = a.ws[a.L.t128_bucket + tile];
    it.start = a.ws[a.L.t128_start + tile];
    it.cnt = min(kMaxTileTokens, a.ws[a.L.offsets + it.bucket + 1] - it.start);
    return it;
}

// Next item of this CTA (stride gridDim.x) at or after `item` whose bucket is a real expert.
template <int MODE>
__device__ inline int next_valid_item(const TcArgs &a, int item, int n_items, int rbs) {
    while (item < n_items && a.ws[a.L.t128_bucket + item / rbs] >= a.E) item += gridDim.x;
    return item;
}

template <int BITS, int G, int MODE>
__global__ void __launch_bounds__(kThreads, 1) grouped_tc_kernel(const TcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the operand tiles (the swizzle pattern repeats every 1024 bytes).
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages], acc_full[1], acc_empty[1], drain_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;
    __shared__ int64_t b_row_off[kBWarps][kMaxTileTokens / kBWarps];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = (int)a.K, n_kb = K / kBK, groups = K / G;
    const int rbs = row_blocks<MODE>(a);
    const int n_items = a.ws[3] * rbs;
    volatile int *abort_v = &abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], kAWarps + (a.x_kind == 3 ? 1 : kBWarps)), mbar_init(&empty_bar[s], kMmaWarps);
        mbar_init(&acc_full[0], kMmaWarps), mbar_init(&acc_empty[0], kEpiWarps);
        mbar_init(&drain_bar, kMmaWarps);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // one warp allocates the CTA's tensor memory (all 512 columns: one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_smem)), "r"(kTmemCols) : "memory");
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

    if (warp >= kFirstAWarp && warp < kFirstBWarp) {
        // ===================== A producers: weights =====================
        // A thread owns one weight row of the item and writes it into its own tensor-memory lane; a warp may only touch
        // the lane quadrant warp % 4, so the row is (accumulator, quadrant, lane).
        const int a_half = (warp - kFirstAWarp) >> 2, a_quad = warp & 3;
        const int p = a_half * 128 + a_quad * 32 + lane;  // weight row of the item, 0..255
        const int64_t row_bytes = BITS == 4 ? a.K / 2 : a.K;
        constexpr int kSuperKb = BITS == 4 ? 4 : 2;  // k-blocks per 128 bytes of packed codes
        constexpr int kWordsPerKb = BITS == 4 ? 8 : 16;
        constexpr int kSuperGroups = (kSuperKb * kBK) / G > 0 ? (kSuperKb * kBK) / G : 1;  // scale groups per super-block
        constexpr int kGroupsPerKb = G >= kBK ? 1 : kBK / G;
        const int n_sb = (n_kb + kSuperKb - 1) / kSuperKb;

        struct Row {
            const uint4 *q;
            const uint16_t *s, *m;
            bool valid;
        };
        auto row_of = [&](int item) {
            Row r{nullptr, nullptr, nullptr, false};
            if (item >= n_items) return r;
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            int64_t wrow;
            if (MODE == kTcSwiglu) {
                const int64_t I = a.N / 2, j = (int64_t)it.rb * 128 + (p & 127);
                r.valid = j < I;
                wrow = (int64_t)it.bucket * a.N + (p < 128 ? j : I + j);
            } else {
                const int64_t rr = (int64_t)it.rb * kAThreads + p;
                r.valid = rr < a.N;
                wrow = (int64_t)it.bucket * a.N + rr;
            }
            r.q = reinterpret_cast<const uint4 *>(a.q + wrow * row_bytes);
            r.s = a.scale + wrow * groups, r.m = a.minv + wrow * groups;
            return r;
        };
        // A super-block: 128 bytes of the row's packed codes (4 k-blocks of Q4, 2 of Q8) and the scales / mins of its
        // groups, fetched one super-block ahead of the one being dequantized - across item boundaries too - so the row
        // is read as whole 128-byte lines and every load has several k-blocks of work to hide behind.
        struct Super {
            uint4 code[8];
            uint32_t sm[kSuperGroups];  // scale | min << 16 (BF16 bits)
        };
        auto load_super = [&](Super &dst, const Row &r, int sb) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dst.code[i] = make_uint4(0u, 0u, 0u, 0u);
                if (r.valid && (sb * kSuperKb + i * kSuperKb / 8) < n_kb) dst.code[i] = __ldg(r.q + sb * 8 + i);
            }
#pragma unroll
            for (int g = 0; g < kSuperGroups; ++g) {
                const int gi = G >= kSuperKb * kBK ? (sb * kSuperKb * kBK) / G : sb * kSuperGroups + g;
                dst.sm[g] = 0u;
                if (r.valid && gi < groups) dst.sm[g] = (uint32_t)__ldg(r.s + gi) | ((uint32_t)__ldg(r.m + gi) << 16);
            }
        };

        uint32_t it_count = 0;  // k-blocks produced so far (stage / phase bookkeeping)
        int item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs);
        Row row = row_of(item);
        Super cur, nxt;
        if (item < n_items) load_super(cur, row, 0);
        bool live = true;
        while (item < n_items && live && !*abort_v) {
            const int next = next_valid_item<MODE>(a, item + gridDim.x, n_items, rbs);
            const Row next_row = row_of(next);
            for (int sb = 0; sb < n_sb && live; ++sb) {
                if (sb + 1 < n_sb) load_super(nxt, row, sb + 1);
                else if (next < n_items) load_super(nxt, next_row, 0);
#pragma unroll
                for (int sub = 0; sub < kSuperKb; ++sub) {
                    const int kb = sb * kSuperKb + sub;
                    if (kb >= n_kb) break;
                    const int stage = it_count % kStages;
                    const uint32_t phase = (it_count / kStages) & 1u;
                    ++it_count;
                    {
                        PROF_BEGIN();
                        if (lane == 0 && !mbar_wait(&empty_bar[stage], phase ^ 1u, abort_v)) raise_abort(item, 1);
                        __syncwarp();
                        if (warp == kFirstAWarp) PROF_ADD(0);
                        if (warp == kFirstAWarp) TRACE(0, it_count - 1, 0);
                    }
                    if (*abort_v) {
                        live = false;
                        break;
                    }
                    PROF_BEGIN();
                    // this thread's row: 64 codes -> 64 F16 = 32 tensor-memory columns of its lane
                    uint32_t words[kWordsPerKb];
#pragma unroll
                    for (int i = 0; i < kWordsPerKb / 4; ++i) {
                        const uint4 v = cur.code[sub * (kWordsPerKb / 4) + i];
                        words[4 * i] = v.x, words[4 * i + 1] = v.y, words[4 * i + 2] = v.z, words[4 * i + 3] = v.w;
                    }
                    __half2 s2[kGroupsPerKb], s16[kGroupsPerKb], m2[kGroupsPerKb];
#pragma unroll
                    for (int gi = 0; gi < kGroupsPerKb; ++gi) {
                        const int g = G >= kSuperKb * kBK ? 0 : (sub * kBK) / G + gi;  // group inside the super-block
                        const uint32_t packed = cur.sm[g < kSuperGroups ? g : 0];
                        const float sf = bf16_bits_to_f32((uint16_t)(packed & 0xffffu)), mf = bf16_bits_to_f32((uint16_t)(packed >> 16));
                        s2[gi] = __float2half2_rn(sf), s16[gi] = __float2half2_rn(sf * 0.0625f), m2[gi] = __float2half2_rn(mf);
                    }
                    const uint32_t a_addr = tmem_base + ((uint32_t)(a_quad * 32) << 16) +
                                            (uint32_t)(kAStageCol0 + stage * kAStageCols + a_half * (kBK / 2));
#pragma unroll
                    for (int hc = 0; hc < 2; ++hc) {  // two stores of 16 columns keep the live registers down
                        uint4 d[4];
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            const int c = hc * 4 + cc;
                            const int gi = kGroupsPerKb == 1 ? 0 : (c * 8) / G;
                            if (BITS == 4) d[cc] = dequant_q4_word(words[c], s2[gi], s16[gi], m2[gi]);
                            else d[cc] = dequant_q8_words(words[2 * c], words[2 * c + 1], s2[gi], m2[gi]);
                        }
                        tc_st16(a_addr + hc * 16, d);
                    }
                    if (warp == kFirstAWarp) PROF_ADD(1);
                    {
                        PROF_BEGIN();
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                        tc_fence_before();  // orders the stores before the MMA warp's reads across the barrier
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&full_bar[stage]);
                        if (warp == kFirstAWarp) TRACE(0, it_count - 1, 1);
                        if (warp == kFirstAWarp) {
                            PROF_ADD(2);
                            PROF_ADD(16 + sub);
                            PROF_COUNT(4);
                        }
                    }
                }
                {
                    PROF_BEGIN();
                    cur = nxt;
#ifdef SXB_TC_PROF
                    asm volatile("" ::"r"(cur.code[7].w), "r"(cur.code[0].x), "r"(cur.sm[0]));
#endif
                    if (warp == kFirstAWarp) PROF_ADD(3);
                }
            }
            item = next;
            row = next_row;
        }
    } else if (warp >= kFirstBWarp) {
        // ===================== B producers: activations =====================
        // B warp w owns tokens [64 w, 64 w + 64) of the tile; lane l copies 16-byte chunk c = l % 8 of tokens
        // 64 w + l / 8 + 4 i (i < 16), every k-block, so eight lanes cover one 128-byte line of one activation row.
        if (a.x_kind == 3) {
            // Tile-blocked activations: one thread, one bulk copy per k-block, completion counted in bytes on the
            // stage's barrier; every free stage is refilled at once, so kStages k-blocks are in flight.
            if (warp == kFirstBWarp && lane == 0) {
                // A second cursor runs kBPrefetch k-blocks ahead of the copies (across items) and pulls those runs into
                // L2, so a copy issued the moment its stage frees up is an L2 hit, not a DRAM round trip.
                uint32_t it_count = 0;
                int p_item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs), p_kb = 0;
                auto prefetch_next = [&]() {
                    if (p_item >= n_items) return;
                    const ItemInfo pi = item_info<MODE>(a, p_item, rbs);
                    const unsigned char *src = reinterpret_cast<const unsigned char *>(a.x) + ((int64_t)p_kb * a.L.S + pi.start) * 128;
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((uint32_t)pi.cnt * 128u) : "memory");
                    if (++p_kb == n_kb) p_kb = 0, p_item = next_valid_item<MODE>(a, p_item + gridDim.x, n_items, rbs);
                };
                for (int i = 0; i < kBPrefetch; ++i) prefetch_next();
                for (int item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs); item < n_items && !*abort_v;
                     item = next_valid_item<MODE>(a, item + gridDim.x, n_items, rbs)) {
                    const ItemInfo it = item_info<MODE>(a, item, rbs);
                    const uint32_t bytes = (uint32_t)it.cnt * 128u;
                    const unsigned char *src = reinterpret_cast<const unsigned char *>(a.x) + (int64_t)it.start * 128;
                    for (int kb = 0; kb < n_kb; ++kb, ++it_count) {
                        prefetch_next();
                        const int stage = it_count % kStages;
                        if (!mbar_wait(&empty_bar[stage], ((it_count / kStages) & 1u) ^ 1u, abort_v)) {
                            raise_abort(item, 5);
                            break;
                        }
                        mbar_expect_tx(&full_bar[stage], bytes);
                        bulk_g2s(smem_u32(smem + stage * kStageBytes), src + (int64_t)kb * a.L.S * 128, bytes, &full_bar[stage]);
                    }
                }
            }
        } else {
        const int bw = warp - kFirstBWarp, c = lane & 7, rg = lane >> 3;
        constexpr int kRowsPerWarp = kMaxTileTokens / kBWarps, kRowsPerLane = kRowsPerWarp / 4;  // 64, 16
        int64_t *row_off = b_row_off[bw];  // element offset of every owned token's activation row (this warp only)
        const bool staged = a.x_kind == 2 || (a.x_kind == 1 && BITS == 8);  // F16 already in this operand's k order
        uint32_t it_count = 0;
        for (int item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs); item < n_items && !*abort_v;
             item = next_valid_item<MODE>(a, item + gridDim.x, n_items, rbs)) {
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            const int n_mine = min(max(it.cnt - bw * kRowsPerWarp, 0), kRowsPerWarp);
            __syncwarp();
            for (int n = lane; n < n_mine; n += 32) {
                const int64_t slot = a.ws[a.L.slots + it.start + bw * kRowsPerWarp + n];
                row_off[n] = (MODE == kTcPartial ? slot : slot / a.A) * a.K;
            }
            __syncwarp();
            bool live = true;
            if (staged) {
                // cp.async straight into the swizzled tile, kBAhead k-blocks in flight; a k-block is handed over when
                // its group has landed (wait_group), behind a proxy fence.
                for (int kb = 0; kb < n_kb + kBAhead && live; ++kb) {
                    // hand over k-block kb - kBAhead first: its group is the oldest of the kBAhead still pending, and the
                    // MMA warp must not have to wait for this warp's next free stage to learn that it has landed
                    if (kb >= kBAhead) {
                        PROF_BEGIN();
                        asm volatile("cp.async.wait_group %0;" ::"n"(kBAhead - 1) : "memory");
                        fence_proxy_async();
                        if (bw == 0) PROF_ADD(14);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&full_bar[(it_count + kb - kBAhead) % kStages]);
                        if (bw == 0) TRACE(1, it_count + kb - kBAhead, 1);
                    }
                    if (kb < n_kb) {
                        const uint32_t cnt = it_count + kb;
                        const int stage = cnt % kStages;
                        {
                            PROF_BEGIN();
                            if (lane == 0 && !mbar_wait(&empty_bar[stage], ((cnt / kStages) & 1u) ^ 1u, abort_v)) raise_abort(item, 5);
                            if (bw == 0) PROF_ADD(12);
                            if (bw == 0) TRACE(1, cnt, 0);
                        }
                        __syncwarp();
                        if (*abort_v) {
                            live = false;
                            break;
                        }
                        const uint32_t sb_ = smem_u32(smem + stage * kStageBytes);
#pragma unroll 4
                        for (int i = 0; i < kRowsPerLane; ++i) {
                            const int nl = rg + 4 * i;
                            if (nl < n_mine)
                                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb_ + swz(bw * kRowsPerWarp + nl, c)),
                                             "l"(a.x + row_off[nl] + kb * kBK + c * 8)
                                             : "memory");
                        }
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            } else {
                // BF16 (or F16 in natural order) activations: through registers, converted and permuted on the way.
                for (int kb = 0; kb < n_kb && live; ++kb) {
                    const uint32_t cnt = it_count + kb;
                    const int stage = cnt % kStages;
                    if (lane == 0 && !mbar_wait(&empty_bar[stage], ((cnt / kStages) & 1u) ^ 1u, abort_v)) raise_abort(item, 5);
                    __syncwarp();
                    if (*abort_v) {
                        live = false;
                        break;
                    }
                    unsigned char *sb_ = smem + stage * kStageBytes;
#pragma unroll 4
                    for (int i = 0; i < kRowsPerLane; ++i) {
                        const int nl = rg + 4 * i;
                        if (nl < n_mine) {
                            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(a.x + row_off[nl] + kb * kBK + c * 8));
                            *reinterpret_cast<uint4 *>(sb_ + swz(bw * kRowsPerWarp + nl, c)) = b_chunk<BITS>(v, a.x_kind == 1);
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_bar[stage]);
                }
            }
            it_count += n_kb;
        }
        }
    } else if (warp >= kMmaWarp) {
        // ===================== MMA issue =====================
        // Two issuing warps, one per accumulator: each instruction costs its issuing thread far more than an N <= 128
        // MMA's arithmetic, so the two halves are issued side by side; a stage is free when both have committed.
        const int half = warp - kMmaWarp;
        uint32_t it_count = 0, acc_count = 0;
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            if (it.bucket >= a.E) continue;
            const uint32_t acc_phase = acc_count & 1u;
            ++acc_count;
            {
                PROF_BEGIN();
                if (lane == 0 && !mbar_wait(&acc_empty[0], acc_phase ^ 1u, abort_v)) raise_abort(item, 2);
                if (half == 0) PROF_ADD(7);
            }
            __syncwarp();
            if (*abort_v) break;
            tc_fence_after();
            const int n_cols = (it.cnt + 15) & ~15;
            const uint32_t idesc = instr_desc(n_cols);
            for (int kb = 0; kb < n_kb; ++kb, ++it_count) {
                const int stage = it_count % kStages;
                const uint32_t phase = (it_count / kStages) & 1u;
                {
                    PROF_BEGIN();
                    if (lane == 0 && !mbar_wait(&full_bar[stage], phase, abort_v)) raise_abort(item, 3);
                    if (half == 0) {
                        PROF_ADD(5);
                        PROF_COUNT(8);
                        TRACE(2, it_count, 0);
                    }
                }
                __syncwarp();
                if (*abort_v) break;
                tc_fence_after();
                PROF_BEGIN();
                if (lane == 0) {
                    const uint32_t sb_ = smem_u32(smem + stage * kStageBytes);
                    const uint32_t d = tmem_base + (uint32_t)(half * kAccCols);
                    const uint32_t at = tmem_base + (uint32_t)(kAStageCol0 + stage * kAStageCols + half * (kBK / 2));
#pragma unroll
                    for (int j = 0; j < kBK / 16; ++j) tc_mma_f16_ts(d, at + j * 8, smem_desc(sb_ + j * 32), idesc, (kb | j) != 0);
                    if (half == 0) PROF_ADD(20);
                    tc_commit(&empty_bar[stage]);                    // frees the stage when these MMAs have read it
                    if (kb == n_kb - 1) tc_commit(&acc_full[0]);     // and hands the accumulators to the epilogue
                }
                if (half == 0) {
                    PROF_ADD(6);
                    TRACE(2, it_count, 1);
                }
                __syncwarp();
            }
        }
        // Drain: every MMA issued by this CTA has completed before tensor memory is released.
        if (lane == 0) {
            tc_commit(&drain_bar);
            mbar_wait(&drain_bar, 0u, abort_v);
        }
        __syncwarp();
    } else {
        // ===================== epilogue =====================
        // Phase 1 (lane = weight row): the finished accumulators are drained from tensor memory into shared memory
        // [accumulator][token][row] and tensor memory is handed back at once - the next item's MMAs run under phase 2.
        // Phase 2: a thread takes one token x 8 consecutive rows, all inside its own warp's 32 rows (no cross-warp
        // dependency): SwiGLU / rounding, then one 16-byte (h, y) or two 16-byte (FP32 partial) stores.
        uint32_t acc_count = 0;
        const int64_t I = a.N / 2;
        float *stage_f = reinterpret_cast<float *>(smem + kStages * kStageBytes);
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            const bool valid = it.bucket < a.E;
            if (valid) {
                const uint32_t acc_phase = acc_count & 1u;
                ++acc_count;
                {
                    PROF_BEGIN();
                    if (lane == 0 && !mbar_wait(&acc_full[0], acc_phase, abort_v)) raise_abort(item, 4);
                    if (warp == 0) {
                        PROF_ADD(9);
                        PROF_COUNT(11);
                    }
                }
                __syncwarp();
                if (*abort_v) break;
                tc_fence_after();
                const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
                for (int c0 = 0; c0 < it.cnt; c0 += 16) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        float v[16];
                        tc_ld16(lane_addr + (uint32_t)(half * kAccCols + c0), v);
                        float *dst = stage_f + ((size_t)half * kMaxTileTokens + c0) * kEpiTokStride + warp * 32 + lane;
#pragma unroll
                        for (int t = 0; t < 16; ++t) dst[t * kEpiTokStride] = v[t];
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[0]);
            }
            PROF_BEGIN();
            const int tl = lane >> 2, g8 = (warp * 32) + (lane & 3) * 8;  // token inside a pass of 8, first of 8 rows
            for (int n = tl; n < it.cnt; n += 8) {
                float r0[8], r1[8];
                if (valid) {
                    const float4 *p0 = reinterpret_cast<const float4 *>(stage_f + (size_t)n * kEpiTokStride + g8);
                    const float4 *p1 = reinterpret_cast<const float4 *>(stage_f + ((size_t)kMaxTileTokens + n) * kEpiTokStride + g8);
                    const float4 x0 = p0[0], x1 = p0[1], y0 = p1[0], y1 = p1[1];
                    r0[0] = x0.x, r0[1] = x0.y, r0[2] = x0.z, r0[3] = x0.w, r0[4] = x1.x, r0[5] = x1.y, r0[6] = x1.z, r0[7] = x1.w;
                    r1[0] = y0.x, r1[1] = y0.y, r1[2] = y0.z, r1[3] = y0.w, r1[4] = y1.x, r1[5] = y1.y, r1[6] = y1.z, r1[7] = y1.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) r0[i] = r1[i] = qnan_f32();
                }
                if (MODE == kTcSwiglu) {
                    const int64_t j = (int64_t)it.rb * 128 + g8;  // h columns j .. j + 7 (I is a multiple of 8)
                    if (j >= I) continue;
                    uint16_t hb[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // kernels/moe_grouped.hip:508-524: from the FP32 accumulators, rounded once
                        const uint16_t b = f32_to_bf16_bits(silu_f32(r0[i]) * r1[i]);
                        hb[i] = a.out_f16 ? __half_as_ushort(__float2half_rn(bf16_bits_to_f32(b))) : b;
                    }
                    uint4 o;
                    if (a.out_f16 == 2 || a.out_f16 == 3) {  // the Q4 operand's k order inside every 8: [0 4 1 5 2 6 3 7]
                        o.x = hb[0] | ((uint32_t)hb[4] << 16), o.y = hb[1] | ((uint32_t)hb[5] << 16);
                        o.z = hb[2] | ((uint32_t)hb[6] << 16), o.w = hb[3] | ((uint32_t)hb[7] << 16);
                    } else {
                        o.x = hb[0] | ((uint32_t)hb[1] << 16), o.y = hb[2] | ((uint32_t)hb[3] << 16);
                        o.z = hb[4] | ((uint32_t)hb[5] << 16), o.w = hb[6] | ((uint32_t)hb[7] << 16);
                    }
                    unsigned char *out = static_cast<unsigned char *>(a.out);
                    if (a.out_f16 >= 3) {
                        *reinterpret_cast<uint4 *>(out + tiled_offset(a.L.S, (int)(j >> 6), it.start + n, n, (int)((j & 63) >> 3))) = o;
                    } else {
                        const int64_t slot = a.ws[a.L.slots + it.start + n];
                        *reinterpret_cast<uint4 *>(out + (slot * I + j) * 2) = o;
                    }
                } else {
                    const int64_t slot = a.ws[a.L.slots + it.start + n];
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int64_t r = (int64_t)it.rb * kAThreads + half * 128 + g8;  // rows r .. r + 7 (N % 8 == 0)
                        const float *v = half ? r1 : r0;
                        if (r >= a.N) continue;
                        if (MODE == kTcPartial) {
                            float4 *o = reinterpret_cast<float4 *>(static_cast<float *>(a.out) + slot * a.N + r);
                            o[0] = make_float4(v[0], v[1], v[2], v[3]);
                            o[1] = make_float4(v[4], v[5], v[6], v[7]);
                        } else {
                            uint4 o;
                            o.x = f32_to_bf16_bits(v[0]) | ((uint32_t)f32_to_bf16_bits(v[1]) << 16);
                            o.y = f32_to_bf16_bits(v[2]) | ((uint32_t)f32_to_bf16_bits(v[3]) << 16);
                            o.z = f32_to_bf16_bits(v[4]) | ((uint32_t)f32_to_bf16_bits(v[5]) << 16);
                            o.w = f32_to_bf16_bits(v[6]) | ((uint32_t)f32_to_bf16_bits(v[7]) << 16);
                            *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(a.out) + slot * a.N + r) = o;
                        }
                    }
                }
            }
            __syncwarp();  // this warp's rows of the staging area are free for its next drain
            if (warp == 0) PROF_ADD(10);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// x [M, K] BF16 -> F16 in the k order of a `bits`-bit weight operand (every 8 consecutive k: [0 4 1 5 2 6 3 7] for
// Q4, natural for Q8): what the B producers would otherwise do per k-block, once per layer instead.
template <int BITS>
__global__ void __launch_bounds__(256) stage_f16_kernel(const uint4 *__restrict__ x, uint4 *__restrict__ xh, int64_t chunks) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (int64_t)gridDim.x * blockDim.x)
        xh[i] = b_chunk<BITS>(x[i], false);
}

// x [M, K] BF16 -> the tile-blocked F16 form (tiled_offset) for the tiles of a grouping workspace: row pos of the
// slot order holds the activation row of token slots[pos] / A, converted, in the operand's k order, swizzled for its place
// in its tile.  One CTA per tile at a time.
template <int BITS>
__global__ void __launch_bounds__(256) stage_tiles_kernel(const uint16_t *__restrict__ x, const int32_t *__restrict__ ws,
                                                          RouteWords L, int64_t A, int64_t K, unsigned char *__restrict__ xs) {
    const int n_tiles = ws[3], chunks_per_row = (int)(K / 8);
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int bucket = ws[L.t128_bucket + tile], start = ws[L.t128_start + tile];
        const int cnt = min(kMaxTileTokens, ws[L.offsets + bucket + 1] - start);
        if (bucket >= L.E) continue;
        // a warp takes one row at a time: its 32 lanes read 512 contiguous bytes of the token's activations per step,
        // four steps in flight
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int n = warp; n < cnt; n += warps) {
            const int64_t tok = ws[L.slots + start + n] / A;
            const uint4 *src = reinterpret_cast<const uint4 *>(x + tok * K);
            for (int k8 = lane; k8 < chunks_per_row; k8 += 128) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (k8 + 32 * u < chunks_per_row) v[u] = src[k8 + 32 * u];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int kk = k8 + 32 * u;
                    if (kk < chunks_per_row)
                        *reinterpret_cast<uint4 *>(xs + tiled_offset(L.S, kk >> 3, start + n, n, kk & 7)) = b_chunk<BITS>(v[u], false);
                }
            }
        }
    }
}

int check_tc(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes, int64_t M,
             int64_t A, const void *out, int act) {
    SXB_CHECK(x != nullptr && out != nullptr && ws != nullptr && w != nullptr, fn, ": null pointer (x=", x, ", out=", out,
              ", ws=", ws, ")");
    SXB_CHECK(w->q != nullptr && w->scale != nullptr && w->minv != nullptr, fn, ": null weight pointer");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->K >= 128 && w->K % 128 == 0 && w->K <= (1 << 24), fn, ": K = ", w->K,
              ", the tcgen05 kernels need a multiple of 128 (two 64-wide k-blocks per 128 bytes of Q8 codes)");
    SXB_CHECK(E >= 1 && E <= kMoeMaxExperts && w->N % E == 0, fn, ": weight has ", w->N, " rows for E = ", E, " experts");
    SXB_CHECK(M >= 1 && A >= 1 && A <= 64 && A <= E && M * A <= kMoeMaxSlots, fn, ": M = ", M, " tokens x A = ", A, " slots");
    SXB_CHECK(ws_bytes >= (size_t)route_words(M, A, E).total * 4, fn, ": workspace of ", ws_bytes, " bytes, needs ",
              route_words(M, A, E).total * 4);
    SXB_CHECK(aligned16(w->q) && aligned16(x), fn, ": code array ", (const void *)w->q, " and input ", x,
              " must be 16-byte aligned");
    SXB_CHECK((w->N / E) % 16 == 0, fn, ": ", w->N / E, " rows an expert, the tcgen05 kernels store 8 rows (SwiGLU: 8 h columns) at a time");
    SXB_CHECK(reinterpret_cast<uintptr_t>(out) % 16 == 0, fn, ": output ", out, " must be 16-byte aligned");
    SXB_CHECK(act == SXB_ACT_BF16 || act == SXB_ACT_F16_STAGED || act == SXB_ACT_F16_TILED, fn,
              ": the WMMA_F16 kernels take BF16 activations (or F16 ones staged by sxb_stage_f16 / sxb_stage_f16_tiles), got ", act);
    return SXB_OK;
}

// The status words of a launch live in the grouping workspace's header (words 5..7, zeroed by the pack).
template <int BITS, int MODE>
int launch_tc(const char *fn, const TcArgs &a, int64_t G, cudaStream_t st) {
    const size_t smem = (size_t)kStages * kStageBytes + kEpiBytes + 1024;
    auto go = [&](auto kern) -> int {
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn,
                 ": reserving shared memory");
        kern<<<(unsigned)sm_count(), kThreads, smem, st>>>(a);
        return SXB_OK;
    };
    switch (G) {
        case 32: return go(grouped_tc_kernel<BITS, 32, MODE>);
        case 64: return go(grouped_tc_kernel<BITS, 64, MODE>);
        default: return go(grouped_tc_kernel<BITS, 128, MODE>);
    }
}

}  // namespace

template <int BITS>
int tc_gather_grouped(const char *fn, const void *x, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes, int64_t M,
                      int64_t A, void *y, int act, bool swiglu, int h_f16, sxb_stream_t stream) {
    if (int rc = check_tc(fn, x, w, E, ws, ws_bytes, M, A, y, act)) return rc;
    const int64_t N = w->N / E;
    SXB_CHECK(!swiglu || N % 2 == 0, fn, ": gate_up has ", N, " rows an expert, expected an even count");
    SXB_CHECK(apart(x, M * w->K * 2, y, M * A * (swiglu ? N / 2 : N) * 2), fn, ": output overlaps input x");
    TcArgs a{};
    a.x = static_cast<const uint16_t *>(x), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = N, a.K = w->K, a.A = A, a.E = E, a.ws = static_cast<const int32_t *>(ws), a.L = route_words(M, A, E);
    a.out = y, a.x_kind = act == SXB_ACT_F16_TILED ? 3 : act == SXB_ACT_F16_STAGED ? 2 : 0, a.out_f16 = h_f16;
    a.status = reinterpret_cast<uint32_t *>(const_cast<void *>(ws)) + 5;
    auto st = static_cast<cudaStream_t>(stream);
    int rc = swiglu ? launch_tc<BITS, kTcSwiglu>(fn, a, w->G, st) : launch_tc<BITS, kTcGather>(fn, a, w->G, st);
    if (rc) return rc;
    SXB_CHECK_LAUNCH(fn, " tcgen05 M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

template <int BITS>
int tc_partial_grouped(const char *fn, const void *h, const SxbQView *w, int64_t E, const void *ws, size_t ws_bytes, int64_t M,
                       int64_t A, float *partial, int act, int h_f16, sxb_stream_t stream) {
    SXB_CHECK((h_f16 != 2 && h_f16 != 3) || BITS == 4, fn, ": h_f16 = ", h_f16, " (the Q4 operand's k order) with a Q8 down weight");
    SXB_CHECK(h_f16 != 4 || BITS == 8, fn, ": h_f16 = 4 (tile-blocked, natural k order) with a Q4 down weight");
    if (int rc = check_tc(fn, h, w, E, ws, ws_bytes, M, A, partial, act)) return rc;
    const int64_t N = w->N / E;
    TcArgs a{};
    a.x = static_cast<const uint16_t *>(h), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = N, a.K = w->K, a.A = A, a.E = E, a.ws = static_cast<const int32_t *>(ws), a.L = route_words(M, A, E);
    a.out = partial, a.x_kind = h_f16 >= 3 ? 3 : h_f16, a.out_f16 = 0;
    a.status = reinterpret_cast<uint32_t *>(const_cast<void *>(ws)) + 5;
    auto st = static_cast<cudaStream_t>(stream);
    if (int rc = launch_tc<BITS, kTcPartial>(fn, a, w->G, st)) return rc;
    SXB_CHECK_LAUNCH(fn, " tcgen05 partial M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

template int tc_gather_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                  void *, int, bool, int, sxb_stream_t);
template int tc_gather_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                  void *, int, bool, int, sxb_stream_t);
template int tc_partial_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                   float *, int, int, sxb_stream_t);
template int tc_partial_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                   float *, int, int, sxb_stream_t);

}  // namespace sxb

extern "C" int sxb_stage_f16_tiles(const void *x, const void *ws, size_t ws_bytes, int64_t M, int64_t A, int64_t E, int64_t K,
                                   int bits, void *xs, sxb_stream_t stream) {
    using namespace sxb;
    SXB_CHECK(x != nullptr && ws != nullptr && xs != nullptr, "stage_f16_tiles: null pointer (x=", x, ", ws=", ws, ", xs=", xs, ")");
    SXB_CHECK(M >= 1 && A >= 1 && A <= 64 && E >= 1 && E <= kMoeMaxExperts && M * A <= kMoeMaxSlots, "stage_f16_tiles: M = ", M,
              ", A = ", A, ", E = ", E);
    SXB_CHECK(K >= 64 && K % 64 == 0, "stage_f16_tiles: K = ", K, " must be a multiple of 64 (one 128-byte line per k-block)");
    SXB_CHECK(bits == 4 || bits == 8, "stage_f16_tiles: k order of a ", bits, "-bit operand unsupported (4 or 8)");
    SXB_CHECK(ws_bytes >= (size_t)route_words(M, A, E).total * 4, "stage_f16_tiles: workspace of ", ws_bytes, " bytes, needs ",
              route_words(M, A, E).total * 4);
    SXB_CHECK(aligned16(x) && aligned16(xs), "stage_f16_tiles: x and xs must be 16-byte aligned");
    const RouteWords L = route_words(M, A, E);
    const unsigned blocks = (unsigned)std::min<int64_t>(L.T128max, (int64_t)sm_count() * 4);
    auto st = static_cast<cudaStream_t>(stream);
    if (bits == 4)
        stage_tiles_kernel<4><<<blocks, 256, 0, st>>>((const uint16_t *)x, (const int32_t *)ws, L, A, K, (unsigned char *)xs);
    else
        stage_tiles_kernel<8><<<blocks, 256, 0, st>>>((const uint16_t *)x, (const int32_t *)ws, L, A, K, (unsigned char *)xs);
    SXB_CHECK_LAUNCH("stage_f16_tiles M=", M, " A=", A, " K=", K, " bits=", bits);
    return SXB_OK;
}

#ifdef SXB_TC_PROF
extern "C" __attribute__((visibility("default"))) int sxb_debug_tc_trace(long long *out) {
    cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(long long) * 4 * 64 * 2);
    return 0;
}
extern "C" __attribute__((visibility("default"))) int sxb_debug_tc_prof(unsigned long long *out, int reset) {
    cudaMemcpyFromSymbol(out, g_tc_prof, sizeof(unsigned long long) * 32);
    if (reset) {
        unsigned long long z[32] = {};
        cudaMemcpyToSymbol(g_tc_prof, z, sizeof(z));
    }
    return 0;
}
#endif

extern "C" int sxb_stage_f16(const void *x, int64_t M, int64_t K, int bits, void *xh, sxb_stream_t stream) {
    using namespace sxb;
    SXB_CHECK(x != nullptr && xh != nullptr, "stage_f16: null pointer (x=", x, ", xh=", xh, ")");
    SXB_CHECK(M >= 1 && K >= 8 && K % 8 == 0, "stage_f16: M = ", M, ", K = ", K, " (K must be a multiple of 8)");
    SXB_CHECK(bits == 4 || bits == 8, "stage_f16: k order of a ", bits, "-bit operand unsupported (4 or 8)");
    SXB_CHECK(aligned16(x) && aligned16(xh), "stage_f16: x and xh must be 16-byte aligned");
    SXB_CHECK(apart(x, M * K * 2, xh, M * K * 2), "stage_f16: xh overlaps x");
    const int64_t chunks = M * K / 8;
    const unsigned blocks = (unsigned)std::min<int64_t>((chunks + 255) / 256, (int64_t)sm_count() * 8);
    auto st = static_cast<cudaStream_t>(stream);
    if (bits == 4) stage_f16_kernel<4><<<blocks, 256, 0, st>>>((const uint4 *)x, (uint4 *)xh, chunks);
    else stage_f16_kernel<8><<<blocks, 256, 0, st>>>((const uint4 *)x, (uint4 *)xh, chunks);
    SXB_CHECK_LAUNCH("stage_f16 M=", M, " K=", K, " bits=", bits);
    return SXB_OK;
}
