// PTX wrappers shared by the tcgen05 kernels of this library (grouped_tc.cu, router_proj.cu): mbarriers with bounded
// waits, bulk / tensor copies into shared memory, tcgen05 MMA issue, commit, tensor-memory loads and stores, and the
// shared-memory / instruction descriptors of kind::f16 MMAs.
#pragma once

#include <cuda.h>  // CUtensorMap and its enums only; the encoder is looked up through the runtime, nothing links libcuda
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace sxb {

// grouped_tc.cu (host): tiled 2-D tensor map; the library's own status words; the current bound of device-side waits.
int tensor_map_2d(const char *fn, const void *base, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner, uint64_t outer,
                  uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle, CUtensorMap *map);
int library_status_words(const char *fn, uint32_t **out);
unsigned long long wait_limit_ns();

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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking: has the phase of this parity completed?  (try_wait may suspend the thread for a while; this never does.)
__device__ inline bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
__device__ inline bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t spins = 0;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 4095u) == 4095u) {
            if (abort_flag != nullptr && *abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}
__device__ inline void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Executed by a whole (converged) warp; elect.sync picks the lane that issues - the same one every time for a full mask,
// so the commits track the MMAs of the lane that issued them.
__device__ inline void tc_commit(uint64_t *bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar))
        : "memory");
}
// 16 consecutive columns of this thread's TMEM lane from each of two addresses, one wait for both.
__device__ inline void tc_ld16x2(uint32_t taddr0, uint32_t taddr1, float (&v0)[16], float (&v1)[16]) {
    uint32_t r[16], q[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr0));
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]), "=r"(q[8]),
          "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15])
        : "r"(taddr1));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v0[i] = __uint_as_float(r[i]), v1[i] = __uint_as_float(q[i]);
}
// silu on the special-function unit: ex2 and a reciprocal, a few ulp of FP32 - far inside the BF16 rounding that follows.
__device__ inline float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// 16 consecutive columns of this thread's TMEM lane, written from registers.
__device__ inline void tc_st16(uint32_t taddr, const uint4 (&d)[4]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(d[0].x), "r"(d[0].y), "r"(d[0].z), "r"(d[0].w), "r"(d[1].x), "r"(d[1].y), "r"(d[1].z), "r"(d[1].w), "r"(d[2].x),
        "r"(d[2].y), "r"(d[2].z), "r"(d[2].w), "r"(d[3].x), "r"(d[3].y), "r"(d[3].z), "r"(d[3].w)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 k of F16, two per 32-bit column) read from tensor memory.
// Whole-warp call, one elected lane issues (see tc_commit).
__device__ inline void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One k-block of an accumulator as one instruction group: a non-blocking probe of the NEXT k-block's "operands ready"
// barrier first, then the four MMAs (k = 16 each; the A columns advance by 8, the B descriptor by 32 bytes), the commit
// that frees the stage and, for the last k-block of an item, the commit that hands the accumulators over.  The probe's
// answer is read only after the commits, so its latency passes under their issue; when it says "ready" the next
// k-block starts without a poll.  Whole-warp call, one elected lane issues.
__device__ inline bool tc_kblock_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                    uint64_t *stage_free, uint64_t *acc_done, uint64_t *next_full, uint32_t next_parity) {
    uint32_t ready;
    asm volatile(
        "{\n\t.reg .pred p, q, r, t, one;\n\t.reg .b32 a1, a2, a3;\n\t.reg .b64 b1, b2, b3;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 r, [%7], %8;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.eq.b32 one, 0, 0;\n\t"
        "add.u32 a1, %2, 8;\n\tadd.u32 a2, %2, 16;\n\tadd.u32 a3, %2, 24;\n\t"
        "add.u64 b1, %3, 2;\n\tadd.u64 b2, %3, 4;\n\tadd.u64 b3, %3, 6;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %4, p;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], b1, %4, one;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a2], b2, %4, one;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a3], b3, %4, one;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
        "setp.ne.b32 t, %9, 0;\n\t"
        "and.pred t, t, q;\n\t"
        "@t tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%9];\n\t"
        "selp.u32 %0, 1, 0, r;\n\t}"
        : "=r"(ready)
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(smem_u32(stage_free)),
          "r"(smem_u32(next_full)), "r"(next_parity), "r"(acc_done ? smem_u32(acc_done) : 0u)
        : "memory");
    return ready != 0;
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

// One box of a 2-D tensor copy, completion counted in bytes on `bar`.  x is a byte offset inside the weight row
// and always a multiple of 64, as the 16-byte alignment rule of tensor copies requires.
__device__ inline void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// 16 bytes global -> shared without passing through registers (both addresses 16-byte aligned); complete, for the
// issuing thread, after cp_async_wait<N> has let at most N of its later groups remain in flight.
__device__ inline void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ inline uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

}  // namespace sxb
