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
// Operands.  A (weights) is read by the MMA from TENSOR MEMORY (the [tmem] form of tcgen05.mma): the producer threads
// dequantize in registers and tcgen05.st the F16 rows straight into their own TMEM lanes, which needs no proxy fence
// (shared-memory operands written by threads do, and that fence cost more than the dequantization).  B (activations)
// is a K-major, 128-byte-swizzled tile in shared memory; with "tile-blocked" activations (sxb_stage_f16_tiles, or the
// h this kernel's own SwiGLU form writes) the tile of a k-block is ONE contiguous run in global memory and arrives by
// one cp.async.bulk.  The packed codes come by 2-D tensor copies (64 bytes x 128 rows a box) into a ring in shared
// memory.  Tensor memory: columns 0-255 the two accumulators, 256-511 four stages of the A operand.
//
// One persistent CTA per SM, 16 warps:
//   warps 0-3   epilogue: tcgen05.ld of the finished accumulators, 16 tokens at a time -> SwiGLU / rounding in
//               registers -> one store per token straight to global memory (a warp's 32 rows of a token are 64 or 128
//               contiguous bytes); tensor memory is handed back as soon as the last columns are in registers
//   warps 4-5   MMA issue, one warp per accumulator (an instruction costs its issuer 60-90 cycles whatever its N);
//               operands warp-uniform, elect.sync picks the issuing lane; tcgen05.commit frees stages / signals
//   warps 6-13  weight producers: a lane quadrant has two warps, which split the k-blocks (even / odd); a thread
//               dequantizes the rows of BOTH accumulators on its lane: lop3 / packed-half arithmetic on 64 codes a
//               row and k-block.  Within every 8 consecutive k both operands use the order [0 4 1 5 2 6 3 7] (Q4),
//               the order in which a nibble pair falls out of one lop3, so no element moves after dequantization
//   warps 14-15 activation producers (one thread issues the bulk copies of tile-blocked activations; the other warp's
//               lane 0 then runs the ring of weight codes; otherwise both warps gather and convert rows)
// Stages are handed over with mbarriers (producers -> MMA: arrive after tcgen05.wait::st; copies: complete_tx bytes;
// MMA -> producers and MMA -> epilogue: tcgen05.commit).  Every wait is bounded: past the limit the CTA raises its abort
// flag, records {2, item, role} in the status words, drains the tensor pipe and frees its tensor memory before returning.
//
// The tensor copies read this GPU's own weight array only, each into the shared memory of the one CTA that issues it.

#include "grouped_tc.cuh"

namespace sxb {
namespace {

// warps 0-3 epilogue, 4-5 MMA issue (one per accumulator), 6-13 weight producers, 14-15 activation producers
constexpr int kEpiWarps = 4, kMmaWarp = 4, kMmaWarps = 2, kFirstAWarp = kMmaWarp + kMmaWarps, kAWarps = 8,
              kFirstBWarp = kFirstAWarp + kAWarps, kBWarps = 2;
constexpr int kThreads = 32 * (kFirstBWarp + kBWarps);  // 512
constexpr int kAThreads = 32 * kAWarps;                 // 256 = weight rows per item
constexpr int kProducers = kAThreads;
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
// Ring of packed weight codes in shared memory: a slot holds 64 bytes (128 Q4 or 64 Q8 codes) of each of the item's 256
// rows, as two boxes of 128 rows.
constexpr int kWSlots = 4;
constexpr int kWSlotBytes = kAThreads * 64;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s: far beyond any legitimate wait (the default bound)

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
    if (a.dense_M > 0) {  // dense projection: tile t holds rows 128 t .. of the one group
        it.bucket = 0, it.start = tile * kMaxTileTokens;
        it.cnt = (int)min((int64_t)kMaxTileTokens, a.dense_M - it.start);
        return it;
    }
    it.bucket = a.ws[a.L.t128_bucket + tile];
    it.start = a.ws[a.L.t128_start + tile];
    it.cnt = min(kMaxTileTokens, a.ws[a.L.offsets + it.bucket + 1] - it.start);
    return it;
}

// Next item of this CTA (stride gridDim.x) at or after `item` whose bucket is a real expert.
template <int MODE>
__device__ inline int next_valid_item(const TcArgs &a, int item, int n_items, int rbs) {
    if (a.dense_M > 0) return item;
    while (item < n_items && a.ws[a.L.t128_bucket + item / rbs] >= a.E) item += gridDim.x;
    return item;
}

template <int BITS, int G, int MODE>
__global__ void __launch_bounds__(kThreads, 1) grouped_tc_kernel(const TcArgs a, const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the operand tiles (the swizzle pattern repeats every 1024 bytes).
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages], acc_full[1], acc_empty[1], drain_bar;
    __shared__ uint64_t w_full[kWSlots], w_empty[kWSlots];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;
    __shared__ int64_t b_row_off[kBWarps][kMaxTileTokens / kBWarps];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = (int)a.K, n_kb = K / kBK, groups = K / G;
    const int rbs = row_blocks<MODE>(a);
    const int n_items = (a.dense_M > 0 ? (int)((a.dense_M + kMaxTileTokens - 1) / kMaxTileTokens) : a.ws[3]) * rbs;
    // slot (row of the output / of h) at position pos of the slot order; a dense projection's rows are in their own order
    auto slot_at = [&](int pos) -> int { return a.dense_M > 0 ? pos : a.ws[a.L.slots + pos]; };
    volatile int *abort_v = &abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], kAWarps / 2 + (a.x_kind == 3 ? 1 : kBWarps)), mbar_init(&empty_bar[s], kMmaWarps);
        mbar_init(&acc_full[0], kMmaWarps), mbar_init(&acc_empty[0], kEpiWarps);
        mbar_init(&drain_bar, kMmaWarps);
        for (int s = 0; s < kWSlots; ++s) mbar_init(&w_full[s], 1), mbar_init(&w_empty[s], BITS == 4 ? kAWarps : kAWarps / 2);
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

    // The ring of weight-code slots is filled by ONE thread.  With tile-blocked activations the second B warp has nothing
    // else to do and its lane 0 runs the ring as far ahead as free slots allow.  Otherwise lane 0 of the first A warp tops
    // the ring up before it consumes slot number j, to slot j + kWSlots - 1, which reuses the buffer of slot j - 1 -
    // released by every A warp as soon as the warp has its codes in registers, so that wait is short.
    constexpr int kKbPerSlot = BITS == 4 ? 2 : 1;  // k-blocks per 64 bytes of packed codes
    const int n_slots = (n_kb + kKbPerSlot - 1) / kKbPerSlot;
    const uint32_t w_base = smem_u32(smem + kStages * kStageBytes);
    const bool own_w_thread = a.x_kind == 3;
    int is_item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs), is_slot = 0, is_y0 = 0, is_y1 = 0;
    uint32_t issued = 0;
    auto issue_one = [&]() -> bool {
        const int slot = issued % kWSlots;
        if (issued >= (uint32_t)kWSlots && !mbar_wait(&w_empty[slot], ((issued / kWSlots) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) {
            raise_abort(is_item, 6);
            return false;
        }
        if (is_slot == 0) {  // the two boxes' first weight rows
            const ItemInfo it = item_info<MODE>(a, is_item, rbs);
            if (MODE == kTcSwiglu) is_y0 = (int)(it.bucket * a.N + it.rb * 128), is_y1 = is_y0 + (int)(a.N / 2);
            else is_y0 = (int)(it.bucket * a.N + (int64_t)it.rb * kAThreads), is_y1 = is_y0 + 128;
        }
        const uint32_t dst = w_base + (uint32_t)(slot * kWSlotBytes);
        // test hook: CTA 0 leaves one slot unfilled (neither the byte count nor the copies), so that its consumers' wait
        // runs out at the launch's limit and the abort path is exercised without anything faulting
        if (!(blockIdx.x == 0 && (int)issued == a.test_skip_slot)) {
            mbar_expect_tx(&w_full[slot], (uint32_t)kWSlotBytes);
            tma_load_2d(dst, &wmap, is_slot * 64, is_y0, &w_full[slot]);
            tma_load_2d(dst + kWSlotBytes / 2, &wmap, is_slot * 64, is_y1, &w_full[slot]);
        }
        ++issued;
        if (++is_slot == n_slots) is_slot = 0, is_item = next_valid_item<MODE>(a, is_item + gridDim.x, n_items, rbs);
        return true;
    };

    if (warp >= kFirstAWarp && warp < kFirstBWarp) {
        // ===================== A producers: weights =====================
        // A thread writes weight rows into its own tensor-memory lane; a warp may only touch the lane quadrant warp % 4.
        // Each quadrant has two producer warps and they split the k-blocks, not the rows: the warp of parity 0 takes the
        // even k-blocks, the other the odd ones, and a thread dequantizes BOTH rows of its lane (accumulator 0's and
        // accumulator 1's).  The two warps that share an SM sub-partition are thereby out of step - while one is in the
        // long dependent chain of barrier polls and hand-over, the other has the arithmetic pipes to itself - and a
        // warp's fixed per-k-block latencies are paid once per two k-blocks of the pipeline.
        // The packed codes arrive in shared memory by tensor copies of 64 bytes x 128 rows (one per accumulator, two per
        // ring slot), so the memory pipe sees a handful of instructions per k-block instead of one 128-byte line per
        // thread: 256 scattered lines per load instruction kept the load/store unit busy for thousands of cycles and
        // held up every other warp's MMA issue.
        const int a_par = (warp - kFirstAWarp) >> 2, a_quad = warp & 3;
        const int p0 = a_quad * 32 + lane;    // row inside either accumulator, 0..127
        constexpr int kKbPerChunk = G / 8;    // k-blocks covered by eight scale groups (one 16-byte load)
        constexpr int kGroupsPerKb = G >= kBK ? 1 : kBK / G;
        constexpr int kCodeRegs = BITS == 4 ? 2 : 4;  // 16-byte chunks of codes per row and k-block
        const bool vec_scales = groups % 8 == 0 && ((reinterpret_cast<uintptr_t>(a.scale) | reinterpret_cast<uintptr_t>(a.minv)) & 15) == 0;
        // this thread's 64 bytes of row p0 inside a box of a slot; 16-byte chunks swizzled (64-byte mode)
        const uint32_t my_w = (uint32_t)(p0 * 64), my_sw = (uint32_t)((p0 >> 1) & 3);

        struct Row {
            int64_t wrow;  // row of the stacked weight
            bool valid;
        };
        auto row_of = [&](int item, int h) {
            Row r{0, false};
            if (item >= n_items) return r;
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            if (MODE == kTcSwiglu) {
                const int64_t I = a.N / 2, j = (int64_t)it.rb * 128 + p0;
                r.valid = j < I;
                r.wrow = (int64_t)it.bucket * a.N + (h == 0 ? j : I + j);
            } else {
                const int64_t rr = (int64_t)it.rb * kAThreads + h * 128 + p0;
                r.valid = rr < a.N;
                r.wrow = (int64_t)it.bucket * a.N + rr;
            }
            return r;
        };
        // Scales and mins of eight consecutive groups of a row (BF16 bits), fetched one chunk ahead of use.
        struct ScaleChunk {
            uint4 s, m;
        };
        auto load_scales = [&](const Row &r, int chunk) {
            ScaleChunk c{make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
            if (!r.valid) return c;
            const int g0 = chunk * 8;
            const uint16_t *sp = a.scale + r.wrow * groups + g0, *mp = a.minv + r.wrow * groups + g0;
            if (vec_scales) {
                c.s = __ldg(reinterpret_cast<const uint4 *>(sp)), c.m = __ldg(reinterpret_cast<const uint4 *>(mp));
            } else {
                uint32_t sw[4] = {0u, 0u, 0u, 0u}, mw[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (g0 + i < groups) sw[i >> 1] |= (uint32_t)__ldg(sp + i) << (16 * (i & 1)), mw[i >> 1] |= (uint32_t)__ldg(mp + i) << (16 * (i & 1));
                c.s = make_uint4(sw[0], sw[1], sw[2], sw[3]), c.m = make_uint4(mw[0], mw[1], mw[2], mw[3]);
            }
            return c;
        };
        auto pick16 = [](const uint4 &v, int g) {
            const uint32_t w = (g & 4) ? ((g & 2) ? v.w : v.z) : ((g & 2) ? v.y : v.x);
            return (uint16_t)((g & 1) ? (w >> 16) : (w & 0xffffu));
        };
        auto top_up = [&](uint32_t upto) {  // lane 0 of the first A warp, when no thread of its own runs the ring
            while (issued < upto + (uint32_t)kWSlots && is_item < n_items)
                if (!issue_one()) break;
        };
        // lane 0: the codes of slot number wc have landed and the stage of k-block number cnt is free
        auto poll = [&](uint32_t wc, uint32_t cnt, int it_for_status) {
            if (!own_w_thread && warp == kFirstAWarp) top_up(wc);
            if (!mbar_wait(&w_full[wc % kWSlots], (wc / kWSlots) & 1u, abort_v, a.wait_limit_ns)) raise_abort(it_for_status, 7);
            else if (!mbar_wait(&empty_bar[cnt % kStages], ((cnt / kStages) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) raise_abort(it_for_status, 1);
        };

        // This warp's k-blocks of an item: kb = a_par, a_par + 2, ...; k-block kb lives in slot kb / kKbPerSlot.
        // Right after the stores of one k-block are issued, lane 0 polls what the warp's NEXT k-block needs, and only then
        // does the warp wait for the stores and hand the k-block over.  The stores' source registers must stay untouched
        // until that wait, hence one row's stores in flight at a time.
        int item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs);
        uint32_t kb_base = 0, w_base_count = 0;  // k-blocks / slots of the items before this one
        Row row[2] = {row_of(item, 0), row_of(item, 1)};
        ScaleChunk sc_cur[2] = {}, sc_nxt[2] = {};
        if (item < n_items) sc_nxt[0] = load_scales(row[0], 0), sc_nxt[1] = load_scales(row[1], 0);
        if (item < n_items && lane == 0) poll((uint32_t)(a_par / kKbPerSlot), (uint32_t)a_par, item);
        __syncwarp();
        bool live = true;
        while (item < n_items && live && !*abort_v) {
            const int next = next_valid_item<MODE>(a, item + gridDim.x, n_items, rbs);
            const Row next_row[2] = {row_of(next, 0), row_of(next, 1)};
            for (int kb = a_par; kb < n_kb; kb += 2) {
                const uint32_t cnt = kb_base + (uint32_t)kb, wc = w_base_count + (uint32_t)(kb / kKbPerSlot);
                const int stage = cnt % kStages, slot = wc % kWSlots;
                if (kb % kKbPerChunk == a_par) {  // this warp's first k-block of a chunk of eight scale groups
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sc_cur[h] = sc_nxt[h];
                        if (kb - a_par + kKbPerChunk < n_kb) sc_nxt[h] = load_scales(row[h], kb / kKbPerChunk + 1);
                        else if (next < n_items) sc_nxt[h] = load_scales(next_row[h], 0);
                    }
                }
                // this k-block's codes of both rows (Q4: half of the slot's 64 bytes of a row; Q8: all of them)
                uint4 code[2][kCodeRegs];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < kCodeRegs; ++c) {
                        const uint32_t chunk = (uint32_t)((BITS == 4 ? (kb & 1) * 2 : 0) + c);
                        code[h][c] = ld_shared_v4(w_base + (uint32_t)(slot * kWSlotBytes + h * (kWSlotBytes / 2)) + my_w + ((chunk ^ my_sw) << 4));
                        if (!row[h].valid) code[h][c] = make_uint4(0u, 0u, 0u, 0u);
                    }
                __syncwarp();
                if (lane == 0) mbar_arrive(&w_empty[slot]);  // the codes are in registers: the slot may be refilled
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    __half2 s2[kGroupsPerKb], s16[kGroupsPerKb], m2[kGroupsPerKb];
#pragma unroll
                    for (int gi = 0; gi < kGroupsPerKb; ++gi) {
                        const int g = ((kb * kBK) / G + gi) & 7;  // group inside the chunk of eight
                        const float sf = bf16_bits_to_f32(pick16(sc_cur[h].s, g)), mf = bf16_bits_to_f32(pick16(sc_cur[h].m, g));
                        s2[gi] = __float2half2_rn(sf), s16[gi] = __float2half2_rn(sf * 0.0625f), m2[gi] = __float2half2_rn(mf);
                    }
                    const uint32_t a_addr = tmem_base + ((uint32_t)(a_quad * 32) << 16) +
                                            (uint32_t)(kAStageCol0 + stage * kAStageCols + h * (kBK / 2));
                    // a row: 64 codes -> 64 F16 = 32 tensor-memory columns of this lane, two stores of 16
#pragma unroll
                    for (int hc = 0; hc < 2; ++hc) {
                        uint4 d[4];
                        if (BITS == 4) {
                            const uint4 v = code[h][hc];  // 32 codes
                            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int cc = 0; cc < 4; ++cc) {
                                const int gi = kGroupsPerKb == 1 ? 0 : ((hc * 4 + cc) * 8) / G;
                                d[cc] = dequant_q4_word(w4[cc], s2[gi], s16[gi], m2[gi]);
                            }
                        } else {
                            const uint4 v0 = code[h][hc * 2], v1 = code[h][hc * 2 + 1];  // 2 x 16 codes
                            const uint32_t w8[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                            for (int cc = 0; cc < 4; ++cc) {
                                const int gi = kGroupsPerKb == 1 ? 0 : ((hc * 4 + cc) * 8) / G;
                                d[cc] = dequant_q8_words(w8[2 * cc], w8[2 * cc + 1], s2[gi], m2[gi]);
                            }
                        }
                        tc_st16(a_addr + hc * 16, d);
                    }
                    if (h == 0) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                {
                    // under the last stores: what this warp's next k-block needs
                    if (lane == 0) {
                        if (kb + 2 < n_kb) poll(w_base_count + (uint32_t)((kb + 2) / kKbPerSlot), cnt + 2, item);
                        else if (next < n_items) poll(w_base_count + (uint32_t)(n_slots + a_par / kKbPerSlot), kb_base + (uint32_t)(n_kb + a_par), next);
                    }
                }
                {
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();  // orders the stores before the MMA warp's reads across the barrier
                    __syncwarp();
                    tc_fence_after();   // and the next k-block's stores after the MMAs that freed its stage
                    if (lane == 0) mbar_arrive(&full_bar[stage]);
                    if (warp == kFirstAWarp) {
                    }
                }
                if (*abort_v) {
                    live = false;
                    break;
                }
            }
            kb_base += (uint32_t)n_kb, w_base_count += (uint32_t)n_slots;
            item = next;
            row[0] = next_row[0], row[1] = next_row[1];
        }
    } else if (warp >= kFirstBWarp) {
        // ===================== B producers: activations =====================
        // B warp w owns tokens [64 w, 64 w + 64) of the tile; lane l copies 16-byte chunk c = l % 8 of tokens
        // 64 w + l / 8 + 4 i (i < 16), every k-block, so eight lanes cover one 128-byte line of one activation row.
        if (a.x_kind == 3) {
            if (warp == kFirstBWarp + 1 && lane == 0)
                while (is_item < n_items && !*abort_v)
                    if (!issue_one()) break;
            // Tile-blocked activations: one thread, one bulk copy per k-block, completion counted in bytes on the
            // stage's barrier; every free stage is refilled at once, so kStages k-blocks are in flight.
            if (warp == kFirstBWarp && lane == 0) {
                uint32_t it_count = 0;
                for (int item = next_valid_item<MODE>(a, blockIdx.x, n_items, rbs); item < n_items && !*abort_v;
                     item = next_valid_item<MODE>(a, item + gridDim.x, n_items, rbs)) {
                    const ItemInfo it = item_info<MODE>(a, item, rbs);
                    const uint32_t bytes = (uint32_t)it.cnt * 128u;
                    const unsigned char *src = reinterpret_cast<const unsigned char *>(a.x) + (int64_t)it.start * 128;
                    for (int kb = 0; kb < n_kb; ++kb, ++it_count) {
                        const int stage = it_count % kStages;
                        if (!mbar_wait(&empty_bar[stage], ((it_count / kStages) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) {
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
                const int64_t slot = slot_at(it.start + bw * kRowsPerWarp + n);
                row_off[n] = (MODE == kTcPartial || MODE == kTcPartialBf16 ? slot : slot / a.A) * a.K;
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
                        asm volatile("cp.async.wait_group %0;" ::"n"(kBAhead - 1) : "memory");
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&full_bar[(it_count + kb - kBAhead) % kStages]);
                    }
                    if (kb < n_kb) {
                        const uint32_t cnt = it_count + kb;
                        const int stage = cnt % kStages;
                        {
                            if (lane == 0 && !mbar_wait(&empty_bar[stage], ((cnt / kStages) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) raise_abort(item, 5);
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
                    if (lane == 0 && !mbar_wait(&empty_bar[stage], ((cnt / kStages) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) raise_abort(item, 5);
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
        // Two issuing warps, one per accumulator: an instruction costs its issuing thread 60-90 cycles whatever its N,
        // more than an N <= 128 MMA's arithmetic, so the two halves are issued side by side; a stage is free when both
        // have committed.  The whole warp runs the loop with warp-uniform operands and elect.sync picks the issuing lane
        // (always the same one for a full mask), which keeps descriptors and addresses out of per-thread registers.
        const int half = __shfl_sync(0xffffffffu, warp, 0) - kMmaWarp;
        const uint32_t d = tmem_base + (uint32_t)(half * kAccCols);
        uint32_t it_count = 0, acc_count = 0;
        bool ready = false;  // the probe issued with the previous k-block already saw this one's operands
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            if (it.bucket >= a.E) continue;
            const uint32_t acc_phase = acc_count & 1u;
            ++acc_count;
            {
                if (lane == 0 && !mbar_wait(&acc_empty[0], acc_phase ^ 1u, abort_v, a.wait_limit_ns)) raise_abort(item, 2);
            }
            __syncwarp();
            if (*abort_v) break;
            tc_fence_after();
            const int n_cols = (it.cnt + 15) & ~15;
            const uint32_t idesc = instr_desc(n_cols);
            for (int kb = 0; kb < n_kb; ++kb, ++it_count) {
                const int stage = it_count % kStages;
                const uint32_t phase = (it_count / kStages) & 1u;
                bool failed = false;
                {
                    if (lane == 0 && !ready && !mbar_wait(&full_bar[stage], phase, abort_v, a.wait_limit_ns)) raise_abort(item, 3), failed = true;
                    if (half == 0) {
                    }
                }
                {
                    // One vote reconverges the warp and tells it whether lane 0's wait gave up (a wait gives up when its
                    // limit runs out or once another warp has raised the abort flag); the item loop re-reads the flag.
                    if (__any_sync(0xffffffffu, failed)) break;
                }
                {
                    tc_fence_after();
                }
                const uint64_t b_desc = smem_desc(smem_u32(smem + stage * kStageBytes));
                const uint32_t at = tmem_base + (uint32_t)(kAStageCol0 + stage * kAStageCols + half * (kBK / 2));
                static_assert(kBK / 16 == 4, "tc_kblock_ts issues four MMAs");
                // the stage is freed when these MMAs have read it; the last k-block hands the accumulators to the epilogue
                ready = tc_kblock_ts(d, at, b_desc, idesc, kb != 0, &empty_bar[stage], kb == n_kb - 1 ? &acc_full[0] : nullptr,
                                     &full_bar[(it_count + 1) % kStages], ((it_count + 1) / kStages) & 1u);
                if (half == 0) {
                }
            }
        }
        // Drain: every MMA issued by this CTA has completed before tensor memory is released.
        // (this wait does not give up when the CTA is aborting: tensor memory must not be released under an MMA)
        tc_commit(&drain_bar);
        if (lane == 0) mbar_wait(&drain_bar, 0u, nullptr, a.wait_limit_ns);
        __syncwarp();
    } else {
        // ===================== epilogue =====================
        // Lane = weight row: 16 tokens of both accumulators at a time from tensor memory into registers; SwiGLU /
        // rounding there (gate row j and up row j of a token sit in the same thread), then one store per token straight
        // to global memory - for a fixed token the warp's 32 rows are 64 (h, y) or 128 (FP32 partial) contiguous bytes,
        // so every store instruction is one line.  Tensor memory goes back to the MMA warps as soon as the last 16
        // tokens are in registers.
        // The per-token code is kept short on purpose (it runs once per item and its instructions are fetched cold):
        // everything that does not depend on the token is folded into per-thread constants; what depends on it - the
        // output row of its slot, or its line in the tile-blocked h - is computed by lanes 0..15 for the 16 tokens of a
        // pass and handed round by shuffles.
        uint32_t acc_count = 0;
        const int64_t I = a.N / 2;
        const int r_loc = warp * 32 + lane;  // row inside a 128-row accumulator
        const bool tiled_out = MODE == kTcSwiglu && a.out_f16 >= 3;
        const bool h_as_f16 = a.out_f16 != 0, q4_order = a.out_f16 == 2 || a.out_f16 == 3;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
            const ItemInfo it = item_info<MODE>(a, item, rbs);
            const bool valid = it.bucket < a.E;
            // per-thread constants of the item: byte offset of this thread's element inside a token's output row / line
            int64_t elem_off;
            uint32_t xor_chunk = 0;  // tile-blocked h: 16-byte chunk of the line, before the per-token swizzle
            bool row_ok;
            if (MODE == kTcSwiglu) {
                const int64_t j = (int64_t)it.rb * 128 + r_loc;  // h column
                const int j7 = (int)(j & 7), pos = q4_order ? (((j7 & 3) << 1) | (j7 >> 2)) : j7;  // [0 4 1 5 2 6 3 7]
                row_ok = j < I;
                if (tiled_out) elem_off = (j >> 6) * a.L.S * 128 + pos * 2, xor_chunk = (uint32_t)((j & 63) >> 3);
                else elem_off = ((j & ~(int64_t)7) + pos) * 2;
            } else {
                const int64_t r = (int64_t)it.rb * kAThreads + r_loc;
                row_ok = r < a.N;  // N is a multiple of 16: the second accumulator's row r + 128 is checked on its own
                elem_off = r * (MODE == kTcPartial ? 4 : 2);
            }
            const bool row1_ok = MODE != kTcSwiglu && (int64_t)it.rb * kAThreads + 128 + r_loc < a.N;
            // Slot of token n of the tile (lanes 0..15 fetch the 16 tokens of a pass, one pass ahead; nothing may depend
            // on the loaded value before the next pass, or the in-order issue would stall this pass's stores behind it).
            auto token_slot = [&](int n) -> int { return (tiled_out || n >= it.cnt) ? 0 : slot_at(it.start + n); };
            // Offset of a token's output row / line, in 16-byte units.
            auto token_off = [&](int n, int slot) -> uint32_t {
                if (tiled_out) return (uint32_t)(it.start + n) * 8u;
                return (uint32_t)(((int64_t)slot * (MODE == kTcSwiglu ? I * 2 : a.N * (MODE == kTcPartial ? 4 : 2))) >> 4);
            };
            int slot_nxt = lane < 16 ? token_slot(lane) : 0;
            if (valid) {
                const uint32_t acc_phase = acc_count & 1u;
                ++acc_count;
                {
                    if (lane == 0 && !mbar_wait(&acc_full[0], acc_phase, abort_v, a.wait_limit_ns)) raise_abort(item, 4);
                    if (warp == 0) {
                    }
                }
                __syncwarp();
                if (*abort_v) break;
                tc_fence_after();
            }
            unsigned char *out = static_cast<unsigned char *>(a.out) + elem_off;
            for (int c0 = 0; c0 < it.cnt; c0 += 16) {
                float g[16], u[16];
                if (valid) {
                    tc_ld16x2(lane_addr + (uint32_t)c0, lane_addr + (uint32_t)(kAccCols + c0), g, u);
                    if (c0 + 16 >= it.cnt) {  // the last columns are out: tensor memory is free for the next item
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[0]);
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 16; ++t) g[t] = u[t] = qnan_f32();
                }
                const uint32_t off_cur = token_off(c0 + (lane & 15), slot_nxt);
                if (c0 + 16 < it.cnt && lane < 16) slot_nxt = token_slot(c0 + 16 + lane);
                const int live = it.cnt - c0;  // tokens of this pass; the columns past them are computed and dropped
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    const int64_t off = (int64_t)__shfl_sync(0xffffffffu, off_cur, t) << 4;
                    if (MODE == kTcSwiglu) {
                        // kernels/moe_grouped.hip:508-524: from the FP32 accumulators, rounded once
                        const uint16_t b = __bfloat16_as_ushort(__float2bfloat16_rn(silu_fast(g[t]) * u[t]));
                        const uint16_t hv = h_as_f16 ? __half_as_ushort(__float2half_rn(bf16_bits_to_f32(b))) : b;
                        const uint32_t sw = tiled_out ? ((xor_chunk ^ (uint32_t)(t & 7)) << 4) : 0u;
                        if (row_ok && t < live) *reinterpret_cast<uint16_t *>(out + off + sw) = hv;
                    } else if (MODE == kTcPartial) {
                        if (row_ok && t < live) *reinterpret_cast<float *>(out + off) = g[t];
                        if (row1_ok && t < live) *reinterpret_cast<float *>(out + off + 512) = u[t];
                    } else {  // BF16 rows: the plain gather's y, or the per-slot dots as kernels/moe_grouped.hip:47-57 stores them
                        if (row_ok && t < live) *reinterpret_cast<uint16_t *>(out + off) = __bfloat16_as_ushort(__float2bfloat16_rn(g[t]));
                        if (row1_ok && t < live) *reinterpret_cast<uint16_t *>(out + off + 256) = __bfloat16_as_ushort(__float2bfloat16_rn(u[t]));
                    }
                }
            }
        }
    }

    // An aborting CTA must not return under copies it issued into its own shared memory (which may go to the next CTA):
    // the thread that ran the ring of weight codes waits, bounded, for the last fill of every slot; the activation copies
    // complete on barriers that also count thread arrivals, so their issuer lets a generous time pass instead.
    if (*abort_v) {
        for (int sl = 0; sl < kWSlots && issued > 0; ++sl) {
            if (issued <= (uint32_t)sl) continue;
            const uint32_t last = ((issued - 1 - (uint32_t)sl) / kWSlots) * kWSlots + (uint32_t)sl;
            if (blockIdx.x == 0 && (int)last == a.test_skip_slot) continue;  // the test hook's slot was never filled
            mbar_wait(&w_full[sl], (last / kWSlots) & 1u, nullptr, 1000000ull);
        }
        if (warp == kFirstBWarp && lane == 0 && a.x_kind == 3)
            for (const unsigned long long t0 = global_ns(); global_ns() - t0 < 50000ull;) {}
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
    // ws == nullptr: a dense projection's rows, in their own order (L.S rows, tile t = rows 128 t ..)
    const int n_tiles = ws ? ws[3] : (int)((L.S + kMaxTileTokens - 1) / kMaxTileTokens), chunks_per_row = (int)(K / 8);
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int bucket = ws ? ws[L.t128_bucket + tile] : 0, start = ws ? ws[L.t128_start + tile] : tile * kMaxTileTokens;
        const int cnt = ws ? min(kMaxTileTokens, ws[L.offsets + bucket + 1] - start) : (int)min((int64_t)kMaxTileTokens, L.S - start);
        if (bucket >= L.E) continue;
        // a warp takes one row at a time: its 32 lanes read 512 contiguous bytes of the token's activations per step,
        // four steps in flight
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int n = warp; n < cnt; n += warps) {
            const int64_t tok = ws ? ws[L.slots + start + n] / A : start + n;
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

// Tensor map over the packed codes of a stacked weight, seen as bytes [rows, row_bytes]: boxes of 64 bytes x 128 rows,
// 16-byte chunks swizzled in the 64-byte mode so that 32 threads reading 32 consecutive rows hit every bank once.
// Rows past the end of the weight read as zero.
int weight_tensor_map(const char *fn, const uint8_t *q, int64_t rows, int64_t row_bytes, CUtensorMap *map) {
    return tensor_map_2d(fn, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)row_bytes, (uint64_t)rows, (uint64_t)row_bytes, 64u, 128u,
                         CU_TENSOR_MAP_SWIZZLE_64B, map);
}

// Knobs of the bounded waits, set through sxb_set_wait_limit / sxb_test_skip_ring_slot and read by every later launch of
// the calling process (plain globals: the library's callers drive it from one thread at a time).
unsigned long long g_wait_limit_ns = kWaitLimitNs;
int g_test_skip_slot = -1;

// Status words of the launches that have no grouping workspace to hold them (dense projections, the router-logits GEMM):
// one set per device, inside the library.
__device__ uint32_t g_dense_status[4];

// The status words of a grouped launch live in the grouping workspace's header (words 5..7, zeroed by the pack).
template <int BITS, int MODE>
int launch_tc(const char *fn, TcArgs a, int64_t G, cudaStream_t st) {
    const size_t smem = (size_t)kStages * kStageBytes + (size_t)kWSlots * kWSlotBytes + 1024;
    a.wait_limit_ns = g_wait_limit_ns, a.test_skip_slot = g_test_skip_slot;
    // Tile-blocked activations have a kernel of their own (grouped_tc_tiled.cu), whose work item is 128 weight rows x up
    // to 192 or 256 tokens.  It wins wherever experts hold many tokens, and for every short contraction (its two
    // accumulators hide the epilogue); a long contraction over experts of a few dozen tokens each is better served by
    // this file's 256 rows per item, since an item costs the same whatever its token count.
    if (a.x_kind == 3) {
        const int64_t per_expert = a.dense_M > 0 ? a.dense_M : a.L.S / a.E;
        if (a.K < 2048 || per_expert >= 160) return launch_tiled_tc<BITS, MODE>(fn, a, G, st);
    }
    CUtensorMap wmap;
    if (int rc = weight_tensor_map(fn, a.q, a.E * a.N, BITS == 4 ? a.K / 2 : a.K, &wmap)) return rc;
    auto go = [&](auto kern) -> int {
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn,
                 ": reserving shared memory");
        kern<<<(unsigned)sm_count(), kThreads, smem, st>>>(a, wmap);
        return SXB_OK;
    };
    switch (G) {
        case 32: return go(grouped_tc_kernel<BITS, 32, MODE>);
        case 64: return go(grouped_tc_kernel<BITS, 64, MODE>);
        default: return go(grouped_tc_kernel<BITS, 128, MODE>);
    }
}

}  // namespace

unsigned long long wait_limit_ns() { return g_wait_limit_ns; }

int library_status_words(const char *fn, uint32_t **out) {
    void *p = nullptr;
    SXB_CUDA(cudaGetSymbolAddress(&p, g_dense_status), fn, ": address of the library's status words");
    *out = static_cast<uint32_t *>(p);
    return SXB_OK;
}

// A 2-D tiled tensor map over row-major data [outer, inner] of `elem_bytes`-byte elements.  The encoder is a host-side
// computation of the driver library, found through the runtime (nothing links libcuda).  Out-of-range parts of a box read
// as zero.
int tensor_map_2d(const char *fn, const void *base, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner, uint64_t outer,
                  uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle, CUtensorMap *map) {
    using TensorMapEncode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                         const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static TensorMapEncode encode = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<TensorMapEncode>(p);
    }();
    SXB_CHECK(encode != nullptr, fn, ": the driver offers no cuTensorMapEncodeTiled");
    (void)elem_bytes;
    const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer}, strides[1] = {(cuuint64_t)row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer}, elem[2] = {1u, 1u};
    const CUresult rc = encode(map, dtype, 2, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SXB_CHECK(rc == CUDA_SUCCESS, fn, ": tensor map over ", outer, " rows of ", row_stride_bytes, " bytes refused (CUresult ", (int)rc, ")");
    return SXB_OK;
}

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
                       int64_t A, float *partial, int act, int h_f16, bool partial_bf16, sxb_stream_t stream) {
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
    if (int rc = partial_bf16 ? launch_tc<BITS, kTcPartialBf16>(fn, a, w->G, st) : launch_tc<BITS, kTcPartial>(fn, a, w->G, st)) return rc;
    SXB_CHECK_LAUNCH(fn, " tcgen05 partial M=", M, " A=", A, " E=", E, " N=", N, " K=", w->K, " G=", w->G);
    return SXB_OK;
}

// A dense projection y [M, N] = x [M, K] * dequant(W)^T on the same kernel: one group, rows in their own order, no
// workspace, and the result written by the epilogue itself (kernels/linear_wmma.hip:69-113).
//   out_kind 0: y BF16;  1: y FP32;  2: W = [gate | up] rows and the output is h = silu(g) * u [M, N / 2], stored as h_f16 says
//   x_kind 0: x BF16 [M, K];  3: x tile-blocked F16 (sxb_stage_f16_tiles with a null workspace)
// status: where a wait that ran out is recorded; null = the library's own words (sxb_check_dense_status).
template <int BITS>
int tc_dense(const char *fn, const void *x, const SxbQView *w, void *y, int64_t M, int x_kind, int out_kind, int h_f16,
             uint32_t *status, sxb_stream_t stream) {
    SXB_CHECK(x != nullptr && y != nullptr && w != nullptr, fn, ": null pointer (x=", x, ", y=", y, ")");
    SXB_CHECK(w->q != nullptr && w->scale != nullptr && w->minv != nullptr, fn, ": null weight pointer");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->K >= 128 && w->K % 128 == 0 && w->K <= (1 << 24), fn, ": K = ", w->K, ", the tcgen05 kernels need a multiple of 128");
    SXB_CHECK(M >= 1 && M <= kMoeMaxSlots, fn, ": M (rows of x) = ", M, ", expected 1..", kMoeMaxSlots);
    SXB_CHECK(w->N >= 16 && w->N % 16 == 0 && w->N <= 0x7fffffff, fn, ": N = ", w->N, " must be a multiple of 16");
    SXB_CHECK(aligned16(w->q) && aligned16(x) && aligned16(y), fn, ": codes, x and y must be 16-byte aligned");
    SXB_CHECK(out_kind != 2 || w->N % 2 == 0, fn, ": [gate | up] rows: N = ", w->N, " must be even");
    const int64_t out_bytes = out_kind == 2 ? M * (w->N / 2) * 2 : M * w->N * (out_kind == 1 ? 4 : 2);
    SXB_CHECK(apart(x, M * w->K * 2, y, out_bytes), fn, ": output y [", y, ", +", out_bytes, " B) overlaps input x [", x, ", +",
              M * w->K * 2, " B)");
    if (status == nullptr)
        if (int rc = library_status_words(fn, &status)) return rc;
    TcArgs a{};
    a.x = static_cast<const uint16_t *>(x), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = w->N, a.K = w->K, a.A = 1, a.E = 1, a.ws = nullptr, a.L = RouteWords{};
    a.L.S = M, a.L.E = 1;
    a.out = y, a.x_kind = x_kind, a.out_f16 = out_kind == 2 ? h_f16 : 0, a.dense_M = M, a.status = status;
    auto st = static_cast<cudaStream_t>(stream);
    int rc = out_kind == 2   ? launch_tc<BITS, kTcSwiglu>(fn, a, w->G, st)
             : out_kind == 1 ? launch_tc<BITS, kTcPartial>(fn, a, w->G, st)
                             : launch_tc<BITS, kTcGather>(fn, a, w->G, st);
    if (rc) return rc;
    SXB_CHECK_LAUNCH(fn, " tcgen05 dense M=", M, " N=", w->N, " K=", w->K, " G=", w->G, " out_kind=", out_kind);
    return SXB_OK;
}

// The up half of the hyper-connection mix as a dense projection with its own epilogue (kTcHcUp): hs = h [M, K] as
// tile-blocked F16, w = W_up's rows in the epilogue's lane order [4 d, K], u [M, d] written by the kernel.
template <int BITS>
int tc_hc_up(const char *fn, const void *hs, const SxbQView *w, const void *x, const float *inv, const float *norm_w, void *u, int64_t M,
             int64_t d, bool f32, sxb_stream_t stream) {
    SXB_CHECK(hs != nullptr && w != nullptr && x != nullptr && inv != nullptr && norm_w != nullptr && u != nullptr, fn, ": null pointer");
    SXB_CHECK(w->G == 32 || w->G == 64 || w->G == 128, fn, ": group size ", w->G, " unsupported (32, 64 or 128)");
    SXB_CHECK(w->K >= 128 && w->K % 128 == 0 && w->K < 2048, fn, ": K = ", w->K, ", expected a multiple of 128 below 2048");
    SXB_CHECK(M >= 1 && M <= kMoeMaxSlots && d >= 32 && d % 32 == 0 && w->N == 4 * d, fn, ": M = ", M, ", d = ", d, ", weight rows ", w->N);
    SXB_CHECK(aligned16(w->q) && aligned16(hs), fn, ": codes and hs must be 16-byte aligned");
    uint32_t *status = nullptr;
    if (int rc = library_status_words(fn, &status)) return rc;
    TcArgs a{};
    a.x = static_cast<const uint16_t *>(hs), a.q = w->q, a.scale = w->scale, a.minv = w->minv;
    a.N = w->N, a.K = w->K, a.A = 1, a.E = 1, a.ws = nullptr, a.L = RouteWords{};
    a.L.S = M, a.L.E = 1;
    a.out = u, a.x_kind = 3, a.out_f16 = 0, a.dense_M = M, a.status = status;
    a.wait_limit_ns = g_wait_limit_ns, a.test_skip_slot = g_test_skip_slot;
    a.hc = TcHcUp{x, inv, norm_w, u, d, f32 ? 1 : 0};
    if (int rc = launch_tiled_tc<BITS, kTcHcUp>(fn, a, w->G, static_cast<cudaStream_t>(stream))) return rc;
    SXB_CHECK_LAUNCH(fn, " tcgen05 up mix M=", M, " d=", d, " K=", w->K, " G=", w->G);
    return SXB_OK;
}
template int tc_hc_up<4>(const char *, const void *, const SxbQView *, const void *, const float *, const float *, void *, int64_t, int64_t, bool,
                         sxb_stream_t);
template int tc_hc_up<8>(const char *, const void *, const SxbQView *, const void *, const float *, const float *, void *, int64_t, int64_t, bool,
                         sxb_stream_t);

template int tc_gather_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                  void *, int, bool, int, sxb_stream_t);
template int tc_gather_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                  void *, int, bool, int, sxb_stream_t);
template int tc_partial_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                   float *, int, int, bool, sxb_stream_t);
template int tc_partial_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                   float *, int, int, bool, sxb_stream_t);
template int tc_dense<4>(const char *, const void *, const SxbQView *, void *, int64_t, int, int, int, uint32_t *, sxb_stream_t);
template int tc_dense<8>(const char *, const void *, const SxbQView *, void *, int64_t, int, int, int, uint32_t *, sxb_stream_t);

}  // namespace sxb

using namespace sxb;

extern "C" int sxb_set_wait_limit(uint64_t nanoseconds) {
    SXB_CHECK(nanoseconds >= 1000ull, "set_wait_limit: ", nanoseconds, " ns is below the minimum of 1000");
    g_wait_limit_ns = nanoseconds;
    return SXB_OK;
}
extern "C" int sxb_test_skip_ring_slot(int slot) {
    g_test_skip_slot = slot;
    return SXB_OK;
}
extern "C" int sxb_check_dense_status(const char *what) {
    uint32_t e[4] = {0, 0, 0, 0};
    SXB_CUDA(cudaMemcpyFromSymbol(e, g_dense_status, sizeof(e)), "check_dense_status: reading the status words");
    if (e[0] == 0) return SXB_OK;
    const uint32_t zero[4] = {0, 0, 0, 0};
    SXB_CUDA(cudaMemcpyToSymbol(g_dense_status, zero, sizeof(zero)), "check_dense_status: clearing the status words");
    return tc_status_error(what, e);
}

// kernels/linear_wmma.hip:69-113 (linear_q4_wmma / linear_q8_wmma): argument rules and dtype pairs of the reference's
// launchers (x 16-byte aligned, y apart from x, out_act == act or BF16 x -> F32 y), BF16 activations only.
namespace {
template <int BITS>
int linear_wmma(const char *fn, const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream) {
    SXB_CHECK(act == SXB_ACT_BF16 || act == SXB_ACT_F16_TILED, fn, ": BF16 activations (or tile-blocked F16 ones) only, got ", act);
    SXB_CHECK(out_act == SXB_ACT_BF16 || out_act == SXB_ACT_F32, fn, ": output dtype ", out_act, " unsupported (BF16 or F32)");
    return tc_dense<BITS>(fn, x, w, y, M, act == SXB_ACT_F16_TILED ? 3 : 0, out_act == SXB_ACT_F32 ? 1 : 0, 0, nullptr, stream);
}
template <int BITS>
int linear_wmma_swiglu(const char *fn, const void *x, const SxbQView *w, void *h, int64_t M, int act, int h_f16, sxb_stream_t stream) {
    SXB_CHECK(act == SXB_ACT_BF16 || act == SXB_ACT_F16_TILED, fn, ": BF16 activations (or tile-blocked F16 ones) only, got ", act);
    SXB_CHECK(h_f16 >= 0 && h_f16 <= 4, fn, ": h_f16 = ", h_f16, ", expected 0..4");
    return tc_dense<BITS>(fn, x, w, h, M, act == SXB_ACT_F16_TILED ? 3 : 0, 2, h_f16, nullptr, stream);
}
}  // namespace
extern "C" int sxb_linear_q4_wmma(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream) {
    return linear_wmma<4>("linear_q4_wmma", x, w, y, M, act, out_act, stream);
}
extern "C" int sxb_linear_q8_wmma(const void *x, const SxbQView *w, void *y, int64_t M, int act, int out_act, sxb_stream_t stream) {
    return linear_wmma<8>("linear_q8_wmma", x, w, y, M, act, out_act, stream);
}
extern "C" int sxb_linear_q4_wmma_swiglu(const void *x, const SxbQView *w, void *h, int64_t M, int act, int h_f16, sxb_stream_t stream) {
    return linear_wmma_swiglu<4>("linear_q4_wmma_swiglu", x, w, h, M, act, h_f16, stream);
}
extern "C" int sxb_linear_q8_wmma_swiglu(const void *x, const SxbQView *w, void *h, int64_t M, int act, int h_f16, sxb_stream_t stream) {
    return linear_wmma_swiglu<8>("linear_q8_wmma_swiglu", x, w, h, M, act, h_f16, stream);
}

extern "C" int sxb_stage_f16_tiles(const void *x, const void *ws, size_t ws_bytes, int64_t M, int64_t A, int64_t E, int64_t K,
                                   int bits, void *xs, sxb_stream_t stream) {
    using namespace sxb;
    SXB_CHECK(x != nullptr && xs != nullptr, "stage_f16_tiles: null pointer (x=", x, ", xs=", xs, ")");
    SXB_CHECK(M >= 1 && A >= 1 && A <= 64 && E >= 1 && E <= kMoeMaxExperts && M * A <= kMoeMaxSlots, "stage_f16_tiles: M = ", M,
              ", A = ", A, ", E = ", E);
    SXB_CHECK(ws != nullptr || (A == 1 && E == 1), "stage_f16_tiles: a null workspace means a dense projection's rows (A = E = 1), got A = ",
              A, ", E = ", E);
    SXB_CHECK(K >= 64 && K % 64 == 0, "stage_f16_tiles: K = ", K, " must be a multiple of 64 (one 128-byte line per k-block)");
    SXB_CHECK(bits == 4 || bits == 8, "stage_f16_tiles: k order of a ", bits, "-bit operand unsupported (4 or 8)");
    SXB_CHECK(ws == nullptr || ws_bytes >= (size_t)route_words(M, A, E).total * 4, "stage_f16_tiles: workspace of ", ws_bytes,
              " bytes, needs ", route_words(M, A, E).total * 4);
    SXB_CHECK(aligned16(x) && aligned16(xs), "stage_f16_tiles: x and xs must be 16-byte aligned");
    RouteWords L = route_words(M, A, E);
    const int64_t tiles = ws ? L.T128max : (M + kMaxTileTokens - 1) / kMaxTileTokens;
    const unsigned blocks = (unsigned)std::min<int64_t>(tiles, (int64_t)sm_count() * 4);
    auto st = static_cast<cudaStream_t>(stream);
    if (bits == 4)
        stage_tiles_kernel<4><<<blocks, 256, 0, st>>>((const uint16_t *)x, (const int32_t *)ws, L, A, K, (unsigned char *)xs);
    else
        stage_tiles_kernel<8><<<blocks, 256, 0, st>>>((const uint16_t *)x, (const int32_t *)ws, L, A, K, (unsigned char *)xs);
    SXB_CHECK_LAUNCH("stage_f16_tiles M=", M, " A=", A, " K=", K, " bits=", bits);
    return SXB_OK;
}

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
