// The tcgen05 expert GEMM for tile-blocked activations (sxb_stage_f16_tiles, or the h that the SwiGLU form of these
// kernels writes): the MoeMath::WmmaF16 forms of linear_q*_experts_gather_grouped[_swiglu] / _combine_grouped
// (kernels/moe_grouped.hpp:58-91) and the dense linear_q*_wmma projections (kernels/linear_wmma.hpp:23-26) when their
// activations arrive in that form.  Numerics as in grouped_tc.cu (kernels/moe_grouped.hpp:29-38,
// kernels/wmma_gemm.hpp:116-129): F16 operands, weights code * scale + min with one rounding, FP32 accumulation.
//
// Why a second kernel.  A k-block of a work item costs about the same whatever the number of tokens it meets: the
// dequantization, the MMA issue and the hand-overs between them are per k-block.  grouped_tc.cu's item is 256 weight
// rows x up to 128 tokens.  Here an item is 128 weight rows (ONE accumulator, a row per tensor-memory lane) x up to 192
// or 256 tokens, so an expert with many tokens has its weights dequantized once per 192 / 256 of them, and the tensor
// memory that the second row half would take holds more pipeline stages or a second accumulator instead:
//   TILE = 256 (long contractions, K >= 2048: gate/up): one accumulator, six stages, three producer warps and two
//              epilogue warps a quadrant;
//   TILE = 192 (short contractions: a down projection is 16 k-blocks): two accumulators - the epilogue of one item runs
//              under the mainloop of the next, which matters most when the mainloop is short - four stages, two
//              producer warps a quadrant.
// The pack cuts both tile lists.  Experts of a few dozen tokens gain nothing from the wider tile and lose the 256 rows per
// item, so the launcher in grouped_tc.cu keeps long contractions over such experts on its own kernel.
//
// SwiGLU: gate row j and up row j are rows of the same accumulator now, so they cannot share a lane.  An item holds 64
// gate rows and their 64 up rows; inside every tensor-memory lane quadrant lanes 0-15 are gate rows and lanes 16-31 the up
// rows of the same h columns, and the epilogue pairs them with one shuffle per value: of the 32 tokens of a pass the gate
// lane finishes the first 16, the up lane the other 16.
//
// Operands as in grouped_tc.cu: A (weights) dequantized in registers and stored to tensor memory by the producer warps
// (the [tmem] form of tcgen05.mma), B (activations) one cp.async.bulk per k-block into a 128-byte-swizzled K-major
// tile, packed codes by 2-D tensor copies (64 bytes x 64 rows a box, two boxes a ring slot).  Tensor memory: the
// accumulator(s) first, then one 32-column A stage per pipeline stage.
//
// One persistent CTA per SM.  Warps: the epilogue first (one per lane quadrant; two per quadrant, each taking half of the
// columns, where there is a single accumulator whose epilogue the MMA warp has to wait for, and in the hyper-connection up
// mix, whose epilogue carries the arithmetic of the stream combine - see TcHcUp), then MMA issue, activation
// copies, the ring of weight codes and one idle warp, then the
// weight producers (a lane quadrant's warps take every second or third k-block each).  A producer hands its k-block
// over before it waits for anything its next one needs.  Every wait is bounded: past the limit the CTA raises its abort
// flag, records {2, item, role} in the status words, drains the tensor pipe and frees its tensor memory before
// returning.  The tensor copies read this GPU's own weight array only, each into the shared memory of the one CTA that
// issues it.

#include "grouped_tc.cuh"

#include <type_traits>

namespace sxb {
namespace {

constexpr int kBK = 64;              // k per stage: one 128-byte swizzle line of F16
constexpr int kRows = 128;           // weight rows per item = tensor-memory lanes
constexpr int kAStageCols = kBK / 2; // 64 F16 of one weight row per lane
constexpr int kTmemCols = 512;
// TILE = tokens per item at most = columns of an accumulator.  Tensor memory holds two accumulators when they fit beside at
// least four A stages (an item's epilogue then runs under the next item's mainloop), else one; the rest is A stages, as
// many as the activation tiles of as many k-blocks fit in shared memory.
// HC: the shape of the hyper-connection up mix (kTcHcUp), whose epilogue does the arithmetic of the stream combine and is
// what its items wait for: a second set of epilogue warps, and a shorter ring of codes (its contractions are a few
// k-blocks) to leave their staging buffers room in shared memory.
template <int TILE, bool HC = false>
struct Shape {
    static constexpr int kAccs = 2 * TILE + 4 * kAStageCols <= kTmemCols ? 2 : 1;
    static constexpr int kStageBytes = TILE * kBK * 2;  // the activation tile of one k-block
    static constexpr int kByTmem = (kTmemCols - kAccs * TILE) / kAStageCols, kBySmem = TILE > 192 ? 6 : 8;
    static constexpr int kStages = kByTmem < kBySmem ? kByTmem : kBySmem;
    static constexpr int kWSlots = TILE > 192 ? 4 : HC ? 6 : 8;  // ring slots of packed codes (8 KB each)
    // Producer warps per lane quadrant: they take every kWays-th k-block each.
    static constexpr int kWays = TILE > 192 ? 3 : 2;
    // Epilogue warps per lane quadrant: a single accumulator's epilogue is exposed (the MMA warp waits for it), so its
    // columns are split between two sets of warps; with two accumulators one set keeps up.
    static constexpr int kEpiSets = kAccs == 1 || HC ? 2 : 1;
    // warps: epilogue | MMA issue, activation copies, ring of weight codes, one idle | producers
    static constexpr int kEpiWarps = 4 * kEpiSets, kMmaWarp = kEpiWarps, kBCopyWarp = kEpiWarps + 1, kWCopyWarp = kEpiWarps + 2,
                         kFirstAWarp = kEpiWarps + 4;
    static constexpr int kThreads = 32 * (kFirstAWarp + 4 * kWays);
    static_assert(TILE % (32 * kEpiSets) == 0 || kEpiSets == 1, "an epilogue set takes whole passes of 32 columns");
    static_assert(TILE % 16 == 0 && TILE <= 256 && kStages > kWays && kStages >= 3, "tile size / pipeline depth");
    static_assert(kStageBytes % 1024 == 0, "operand tiles start on the swizzle pattern's 1024-byte period");
};
constexpr int kWSlotBytes = kRows * 64;  // 64 bytes (128 Q4 or 64 Q8 codes) of each of the item's rows
// kTcHcUp: one buffer of an epilogue warp - a pass's 128 (token, stream) segments of X, 32 bytes each at most, then inv
constexpr int kHcUpBufBytes = 128 * 32 + 32 * 16;

struct Item {
    int bucket, start, cnt;  // expert (bucket E = invalid ids), first position in slots[], tokens of the item
    int rb;                  // row block
};

template <int MODE>
__device__ inline int row_blocks(const TcArgs &a) {
    return MODE == kTcSwiglu ? (int)((a.N / 2 + kRows / 2 - 1) / (kRows / 2)) : (int)((a.N + kRows - 1) / kRows);
}
template <int TILE>
__device__ inline int tile_count(const TcArgs &a) {
    static_assert(TILE == kTcTileA || TILE == kTcTileB, "the pack cuts tiles of these two sizes");
    if (a.dense_M > 0) return (int)((a.dense_M + TILE - 1) / TILE);
    return a.ws[TILE == kTcTileA ? a.L.tta_n : a.L.ttb_n];
}
template <int TILE>
__device__ inline Item item_info(const TcArgs &a, int item, int rbs) {
    constexpr int kTile = TILE;
    Item it;
    const int tile = item / rbs;
    it.rb = item % rbs;
    if (a.dense_M > 0) {  // dense projection: tile t holds rows kTile * t .. of the one group
        it.bucket = 0, it.start = tile * kTile;
        it.cnt = (int)min((int64_t)kTile, a.dense_M - it.start);
        return it;
    }
    it.bucket = a.ws[(TILE == kTcTileA ? a.L.tta_bucket : a.L.ttb_bucket) + tile];
    it.start = a.ws[(TILE == kTcTileA ? a.L.tta_start : a.L.ttb_start) + tile];
    it.cnt = min(kTile, a.ws[a.L.offsets + it.bucket + 1] - it.start);
    return it;
}
// Next item of this CTA (stride gridDim.x) at or after `item` whose bucket is a real expert.
template <int TILE>
__device__ inline int next_valid_item(const TcArgs &a, int item, int n_items, int rbs) {
    if (a.dense_M > 0) return item;
    const int64_t tb = TILE == kTcTileA ? a.L.tta_bucket : a.L.ttb_bucket;
    while (item < n_items && a.ws[tb + item / rbs] >= a.E) item += gridDim.x;
    return item;
}

template <int BITS, int G, int MODE, int TILE>
__global__ void __launch_bounds__((Shape<TILE, MODE == kTcHcUp>::kThreads), 1)
    tiled_tc_kernel(const TcArgs a, const __grid_constant__ CUtensorMap wmap) {
    using S = Shape<TILE, MODE == kTcHcUp>;
    constexpr int kTile = TILE, kAccs = S::kAccs, kStages = S::kStages, kStageBytes = S::kStageBytes, kWSlots = S::kWSlots, kWays = S::kWays,
                  kEpiSets = S::kEpiSets, kEpiWarps = S::kEpiWarps, kMmaWarp = S::kMmaWarp, kBCopyWarp = S::kBCopyWarp,
                  kWCopyWarp = S::kWCopyWarp, kFirstAWarp = S::kFirstAWarp;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the operand tiles (the swizzle pattern repeats every 1024 bytes).
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages], acc_full[2], acc_empty[2], drain_bar;
    __shared__ uint64_t w_full[kWSlots], w_empty[kWSlots];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = (int)a.K, n_kb = K / kBK, groups = K / G;
    const int rbs = row_blocks<MODE>(a);
    const int n_items = tile_count<TILE>(a) * rbs;
    // slot (row of the output / of h) at position pos of the slot order; a dense projection's rows are in their own order
    auto slot_at = [&](int pos) -> int { return a.dense_M > 0 ? pos : a.ws[a.L.slots + pos]; };
    volatile int *abort_v = &abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 4 + 1), mbar_init(&empty_bar[s], 1);
        for (int h = 0; h < kAccs; ++h) mbar_init(&acc_full[h], 1), mbar_init(&acc_empty[h], kEpiWarps);
        mbar_init(&drain_bar, 1);
        for (int s = 0; s < kWSlots; ++s) mbar_init(&w_full[s], 1), mbar_init(&w_empty[s], BITS == 4 ? 8 : 4);
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

    constexpr int kKbPerSlot = BITS == 4 ? 2 : 1;  // k-blocks per 64 bytes of packed codes
    const int n_slots = (n_kb + kKbPerSlot - 1) / kKbPerSlot;
    const uint32_t w_base = smem_u32(smem + kStages * kStageBytes);
    uint32_t issued = 0;  // ring slots issued by this thread (the ring's thread only)

    if (warp >= kFirstAWarp && (warp - kFirstAWarp) >> 2 < n_kb) {
        // ===================== A producers: weights =====================
        // A thread writes one weight row into its own tensor-memory lane; a warp may only touch the lane quadrant
        // warp % 4.  The kWays warps of a quadrant take every kWays-th k-block each, so that while one is in its chain of
        // barrier polls and hand-over the others have the arithmetic pipes, and a warp's fixed per-k-block latencies are
        // paid once per kWays k-blocks of the pipeline.
        const int a_par = (warp - kFirstAWarp) >> 2, a_quad = warp & 3;  // a_par: which of every kWays k-blocks
        const int p0 = a_quad * 32 + lane;  // tensor-memory lane = row of the item
        // row of the ring slot that holds this lane's codes: the SwiGLU form's slot is [64 gate rows | 64 up rows]
        const int srow = MODE == kTcSwiglu ? (lane >> 4) * (kRows / 2) + a_quad * 16 + (lane & 15) : p0;
        constexpr int kKbPerChunk = G / 8;  // k-blocks covered by eight scale groups (one 16-byte load)
        static_assert(kWays <= kKbPerChunk, "a warp's consecutive k-blocks never skip a chunk of scale groups");
        constexpr int kGroupsPerKb = G >= kBK ? 1 : kBK / G;
        constexpr int kCodeRegs = BITS == 4 ? 2 : 4;  // 16-byte chunks of codes per row and k-block
        const bool vec_scales = groups % 8 == 0 && ((reinterpret_cast<uintptr_t>(a.scale) | reinterpret_cast<uintptr_t>(a.minv)) & 15) == 0;
        // this thread's 64 bytes inside a slot; 16-byte chunks swizzled (64-byte mode)
        const uint32_t my_w = (uint32_t)(srow * 64), my_sw = (uint32_t)((srow >> 1) & 3);

        struct Row {
            int64_t wrow;  // row of the stacked weight
            bool valid;
        };
        auto row_of = [&](int item) {
            Row r{0, false};
            if (item >= n_items) return r;
            const Item it = item_info<TILE>(a, item, rbs);
            if (MODE == kTcSwiglu) {
                const int64_t I = a.N / 2, j = (int64_t)it.rb * (kRows / 2) + a_quad * 16 + (lane & 15);
                r.valid = j < I;
                r.wrow = (int64_t)it.bucket * a.N + ((lane >> 4) ? I + j : j);
            } else {
                const int64_t rr = (int64_t)it.rb * kRows + p0;
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
        // lane 0: the codes of slot number wc have landed and the stage of k-block number cnt is free
        auto poll = [&](uint32_t wc, uint32_t cnt, int it_for_status) {
            if (!mbar_wait(&w_full[wc % kWSlots], (wc / kWSlots) & 1u, abort_v, a.wait_limit_ns)) {
                raise_abort(it_for_status, 7);
                return;
            }
            if (!mbar_wait(&empty_bar[cnt % kStages], ((cnt / kStages) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) raise_abort(it_for_status, 1);
        };

        // This warp's k-blocks of an item: kb = a_par, a_par + kWays, ...; k-block kb lives in slot kb / kKbPerSlot.  The
        // stores' source registers must stay untouched until tcgen05.wait::st.
        int item = next_valid_item<TILE>(a, blockIdx.x, n_items, rbs);
        uint32_t kb_base = 0, w_base_count = 0;  // k-blocks / slots of the items before this one
        Row row = row_of(item);
        ScaleChunk sc_cur = {}, sc_nxt = {};
        if (item < n_items) sc_nxt = load_scales(row, 0);
        if (item < n_items && lane == 0) poll((uint32_t)(a_par / kKbPerSlot), (uint32_t)a_par, item);
        __syncwarp();
        bool live = true;
        while (item < n_items && live && !*abort_v) {
            const int next = next_valid_item<TILE>(a, item + gridDim.x, n_items, rbs);
            const Row next_row = row_of(next);
            int cur_chunk = -1;
            for (int kb = a_par; kb < n_kb; kb += kWays) {
                const uint32_t cnt = kb_base + (uint32_t)kb, wc = w_base_count + (uint32_t)(kb / kKbPerSlot);
                const int stage = cnt % kStages, slot = wc % kWSlots;
                if (kb / kKbPerChunk != cur_chunk) {  // this warp's first k-block in a chunk of eight scale groups
                    cur_chunk = kb / kKbPerChunk;
                    sc_cur = sc_nxt;
                    int nkb = kb + kWays;  // this warp's first k-block past the chunk (kWays <= kKbPerChunk: no chunk is skipped)
                    while (nkb / kKbPerChunk == cur_chunk) nkb += kWays;
                    if (nkb < n_kb) sc_nxt = load_scales(row, nkb / kKbPerChunk);
                    else if (next < n_items) sc_nxt = load_scales(next_row, 0);
                }
                // this k-block's codes of the row (Q4: half of the slot's 64 bytes of a row; Q8: all of them)
                uint4 code[kCodeRegs];
#pragma unroll
                for (int c = 0; c < kCodeRegs; ++c) {
                    const uint32_t chunk = (uint32_t)((BITS == 4 ? (kb & 1) * 2 : 0) + c);
                    code[c] = ld_shared_v4(w_base + (uint32_t)(slot * kWSlotBytes) + my_w + ((chunk ^ my_sw) << 4));
                    if (!row.valid) code[c] = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&w_empty[slot]);  // the codes are in registers: the slot may be refilled
                __half2 s2[kGroupsPerKb], s16[kGroupsPerKb], m2[kGroupsPerKb];
#pragma unroll
                for (int gi = 0; gi < kGroupsPerKb; ++gi) {
                    const int g = ((kb * kBK) / G + gi) & 7;  // group inside the chunk of eight
                    const float sf = bf16_bits_to_f32(pick16(sc_cur.s, g)), mf = bf16_bits_to_f32(pick16(sc_cur.m, g));
                    s2[gi] = __float2half2_rn(sf), s16[gi] = __float2half2_rn(sf * 0.0625f), m2[gi] = __float2half2_rn(mf);
                }
                const uint32_t a_addr = tmem_base + ((uint32_t)(a_quad * 32) << 16) + (uint32_t)(kAccs * kTile + stage * kAStageCols);
                // the row: 64 codes -> 64 F16 = 32 tensor-memory columns of this lane, two stores of 16
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    uint4 d[4];
                    if (BITS == 4) {
                        const uint4 v = code[hc];  // 32 codes
                        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            const int gi = kGroupsPerKb == 1 ? 0 : ((hc * 4 + cc) * 8) / G;
                            d[cc] = dequant_q4_word(w4[cc], s2[gi], s16[gi], m2[gi]);
                        }
                    } else {
                        const uint4 v0 = code[hc * 2], v1 = code[hc * 2 + 1];  // 2 x 16 codes
                        const uint32_t w8[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            const int gi = kGroupsPerKb == 1 ? 0 : ((hc * 4 + cc) * 8) / G;
                            d[cc] = dequant_q8_words(w8[2 * cc], w8[2 * cc + 1], s2[gi], m2[gi]);
                        }
                    }
                    tc_st16(a_addr + hc * 16, d);
                }
                // Under the stores: a look (never a wait) at what this warp's next k-block needs - its codes landed, its
                // stage free.  The k-block in hand is handed over BEFORE any wait for those: a producer that waited for a
                // free stage while holding back a finished k-block would tie the MMA warp's progress to its own.
                uint32_t nwc = 0, ncnt = 0;
                int nitem = -1;  // -1: this warp has no further k-block
                if (kb + kWays < n_kb) nwc = w_base_count + (uint32_t)((kb + kWays) / kKbPerSlot), ncnt = cnt + kWays, nitem = item;
                else if (next < n_items) nwc = w_base_count + (uint32_t)(n_slots + a_par / kKbPerSlot), ncnt = kb_base + (uint32_t)(n_kb + a_par), nitem = next;
                bool seen = true;
                if (lane == 0 && nitem >= 0)
                    seen = mbar_test_wait(&w_full[nwc % kWSlots], (nwc / kWSlots) & 1u) &&
                           mbar_test_wait(&empty_bar[ncnt % kStages], ((ncnt / kStages) & 1u) ^ 1u);
                __syncwarp();
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();  // orders the stores before the MMA warp's reads across the barrier
                __syncwarp();
                tc_fence_after();   // and the next k-block's stores after the MMAs that freed its stage
                if (lane == 0) {
                    mbar_arrive(&full_bar[stage]);
                    if (!seen) poll(nwc, ncnt, nitem);
                }
                __syncwarp();
                if (*abort_v) {
                    live = false;
                    break;
                }
            }
            kb_base += (uint32_t)n_kb, w_base_count += (uint32_t)n_slots;
            item = next;
            row = next_row;
        }
    } else if (warp == kWCopyWarp) {
        // ===================== the ring of weight codes =====================
        // One thread keeps the ring as far ahead as free slots allow: per slot two boxes of 64 rows (the SwiGLU form: the
        // gate rows and, I rows further, their up rows; otherwise 128 consecutive rows).
        if (lane == 0) {
            int is_item = next_valid_item<TILE>(a, blockIdx.x, n_items, rbs), is_slot = 0, y0 = 0, y1 = 0;
            while (is_item < n_items && !*abort_v) {
                const int slot = issued % kWSlots;
                if (issued >= (uint32_t)kWSlots && !mbar_wait(&w_empty[slot], ((issued / kWSlots) & 1u) ^ 1u, abort_v, a.wait_limit_ns)) {
                    raise_abort(is_item, 6);
                    break;
                }
                if (is_slot == 0) {
                    const Item it = item_info<TILE>(a, is_item, rbs);
                    if (MODE == kTcSwiglu) y0 = (int)(it.bucket * a.N + it.rb * (kRows / 2)), y1 = y0 + (int)(a.N / 2);
                    else y0 = (int)(it.bucket * a.N + (int64_t)it.rb * kRows), y1 = y0 + kRows / 2;
                }
                const uint32_t dst = w_base + (uint32_t)(slot * kWSlotBytes);
                // test hook: CTA 0 leaves one slot unfilled (neither the byte count nor the copies), so that its consumers'
                // wait runs out at the launch's limit and the abort path is exercised without anything faulting
                if (!(blockIdx.x == 0 && (int)issued == a.test_skip_slot)) {
                    mbar_expect_tx(&w_full[slot], (uint32_t)kWSlotBytes);
                    tma_load_2d(dst, &wmap, is_slot * 64, y0, &w_full[slot]);
                    tma_load_2d(dst + kWSlotBytes / 2, &wmap, is_slot * 64, y1, &w_full[slot]);
                }
                ++issued;
                if (++is_slot == n_slots) is_slot = 0, is_item = next_valid_item<TILE>(a, is_item + gridDim.x, n_items, rbs);
            }
        }
    } else if (warp == kBCopyWarp) {
        // ===================== activations =====================
        // One thread, one bulk copy per k-block: the tile of (item, k-block) is one contiguous run of cnt * 128 bytes;
        // completion is counted in bytes on the stage's barrier, and every free stage is refilled at once.
        if (lane == 0) {
            uint32_t it_count = 0;
            for (int item = next_valid_item<TILE>(a, blockIdx.x, n_items, rbs); item < n_items && !*abort_v;
                 item = next_valid_item<TILE>(a, item + gridDim.x, n_items, rbs)) {
                const Item it = item_info<TILE>(a, item, rbs);
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
    } else if (warp == kMmaWarp) {
        // ===================== MMA issue =====================
        // The whole warp runs the loop with warp-uniform operands and elect.sync picks the issuing lane (always the same
        // one for a full mask), which keeps descriptors and addresses out of per-thread registers.
        uint32_t it_count = 0, acc_count = 0;
        bool ready = false;  // the probe issued with the previous k-block already saw this one's operands
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
            const Item it = item_info<TILE>(a, item, rbs);
            if (it.bucket >= a.E) continue;
            const uint32_t half = acc_count % kAccs, acc_phase = (acc_count / kAccs) & 1u;  // the accumulators take turns
            ++acc_count;
            if (lane == 0 && !mbar_wait(&acc_empty[half], acc_phase ^ 1u, abort_v, a.wait_limit_ns)) raise_abort(item, 2);
            __syncwarp();
            if (*abort_v) break;
            tc_fence_after();
            const int n_cols = (it.cnt + 15) & ~15;
            const uint32_t idesc = instr_desc(n_cols);
            const uint32_t d = tmem_base + half * (uint32_t)kTile;
            for (int kb = 0; kb < n_kb; ++kb, ++it_count) {
                const int stage = it_count % kStages;
                const uint32_t phase = (it_count / kStages) & 1u;
                bool failed = false;
                if (lane == 0 && !ready && !mbar_wait(&full_bar[stage], phase, abort_v, a.wait_limit_ns)) raise_abort(item, 3), failed = true;
                // One vote reconverges the warp and tells it whether lane 0's wait gave up (a wait gives up when its
                // limit runs out or once another warp has raised the abort flag); the item loop re-reads the flag.
                if (__any_sync(0xffffffffu, failed)) break;
                tc_fence_after();
                const uint64_t b_desc = smem_desc(smem_u32(smem + stage * kStageBytes));
                const uint32_t at = tmem_base + (uint32_t)(kAccs * kTile + stage * kAStageCols);
                static_assert(kBK / 16 == 4, "tc_kblock_ts issues four MMAs");
                // the stage is freed when these MMAs have read it; the last k-block hands the accumulator to the epilogue
                const bool last = kb == n_kb - 1;
                ready = tc_kblock_ts(d, at, b_desc, idesc, kb != 0, &empty_bar[stage], last ? &acc_full[half] : nullptr,
                                     &full_bar[(it_count + 1) % kStages], ((it_count + 1) / kStages) & 1u);
            }
        }
        // Drain: every MMA issued by this CTA has completed before tensor memory is released.
        // (this wait does not give up when the CTA is aborting: tensor memory must not be released under an MMA)
        tc_commit(&drain_bar);
        if (lane == 0) mbar_wait(&drain_bar, 0u, nullptr, a.wait_limit_ns);
        __syncwarp();
    } else if (MODE == kTcHcUp && warp < kEpiWarps) {
        // ===================== epilogue of the hyper-connection up mix =====================
        // Lane = (stream s = lane & 3, output column j): per token it needs one activation X[t, s d + j] and inv[t, s].
        // Loads into registers would stall the in-order issue once per token, so a pass's 32 tokens x 4 streams x 8 columns
        // of X and 32 x 4 of inv come through shared memory by 16-byte asynchronous copies (no registers held), issued one
        // pass ahead - across items too - into the warp's own double buffer.  Same hand-overs with the MMA warp as below.
        if constexpr (MODE == kTcHcUp) {
            // The activation dtype is a compile-time constant of the loops (one instantiation each): a run-time choice
            // between two loads per token would put a branch between the tokens, and their chains would not overlap.
            auto run = [&](auto f32_tag) {
                constexpr bool kF32 = decltype(f32_tag)::value;
                constexpr int es = kF32 ? 4 : 2, seg = 8 * es;  // bytes of a (token, stream) segment: this quadrant's 8 columns
                constexpr int kPieces = (128 * seg / 16) / 32;   // 16-byte copies per lane and pass
                using TX = typename std::conditional<kF32, float, uint16_t>::type;
                const TcHcUp &hc = a.hc;
                uint32_t acc_count = 0, pass_count = 0;
                const int quad = warp & 3, s = lane & 3, jj = lane >> 2;
                const int col_lo = (warp >> 2) * (kTile / kEpiSets);
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
                const int64_t row_bytes = 4 * hc.d * es;  // a token's four streams
                unsigned char *my_buf = smem + kStages * kStageBytes + kWSlots * kWSlotBytes + warp * (2 * kHcUpBufBytes);
                // Copy number k of a pass: piece p = 32 k + lane of the pass's [token][stream][part] order, i.e. token
                // k * (8 / parts) + tok_l, stream str_l, part part_l with parts = seg / 16.
                constexpr int kParts = seg / 16, kTokStep = 8 / kParts;
                const int part_l = lane % kParts, str_l = (lane / kParts) & 3, tok_l = lane / (4 * kParts);
                auto issue = [&](const Item &it, int c0, int col_hi, unsigned char *buf) {
                    const unsigned char *src = static_cast<const unsigned char *>(hc.x) + ((int64_t)it.rb * 32 + quad * 8 + (int64_t)str_l * hc.d) * es +
                                               part_l * 16 + (int64_t)(it.start + c0 + tok_l) * row_bytes;
                    const uint32_t dst = smem_u32(buf) + (uint32_t)lane * 16u;
#pragma unroll
                    for (int k = 0; k < kPieces; ++k)
                        if (c0 + k * kTokStep + tok_l < col_hi) cp_async16(dst + (uint32_t)k * 512u, src + (int64_t)(k * kTokStep) * row_bytes);
                    if (c0 + lane < col_hi) cp_async16(smem_u32(buf) + 128 * 32 + (uint32_t)lane * 16u, hc.inv + (int64_t)(it.start + c0 + lane) * 4);
                    cp_async_commit();
                };
                auto col_hi_of = [&](const Item &it) { return min(it.cnt, col_lo + kTile / kEpiSets); };
                if (blockIdx.x < n_items) {
                    const Item it0 = item_info<TILE>(a, blockIdx.x, rbs);
                    issue(it0, col_lo, col_hi_of(it0), my_buf);
                }
                for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
                    const Item it = item_info<TILE>(a, item, rbs);
                    const int64_t j = (int64_t)it.rb * 32 + quad * 8 + jj;
                    const float nwp = 1.0f + __ldg(hc.norm_w + (int64_t)s * hc.d + j);
                    const int col_hi = col_hi_of(it);
                    const uint32_t half = acc_count % kAccs, acc_phase = (acc_count / kAccs) & 1u;
                    ++acc_count;
                    if (lane == 0 && !mbar_wait(&acc_full[half], acc_phase, abort_v, a.wait_limit_ns)) raise_abort(item, 4);
                    __syncwarp();
                    if (*abort_v) break;
                    tc_fence_after();
                    if (col_lo >= col_hi && lane == 0) mbar_arrive(&acc_empty[half]);
                    // a pass is issued even when this set has no tokens in the item, so that every item consumes one buffer at least
                    for (int c0 = col_lo; c0 < col_hi || c0 == col_lo; c0 += 32) {
                        unsigned char *buf = my_buf + (pass_count & 1u) * kHcUpBufBytes, *nxt = my_buf + ((pass_count + 1) & 1u) * kHcUpBufBytes;
                        ++pass_count;
                        __syncwarp();  // every lane has finished reading the buffer that the next copies overwrite
                        if (c0 + 32 < col_hi) {
                            issue(it, c0 + 32, col_hi, nxt);
                        } else if (item + (int)gridDim.x < n_items) {
                            const Item itn = item_info<TILE>(a, item + gridDim.x, rbs);
                            issue(itn, col_lo, col_hi_of(itn), nxt);
                        } else {
                            cp_async_commit();
                        }
                        if (c0 >= col_hi) {  // nothing to finish: only the buffer rotation above
                            cp_async_wait<1>();
                            break;
                        }
                        float va[16], vb[16];
                        const uint32_t tcol = lane_addr + half * (uint32_t)kTile + (uint32_t)c0;
                        tc_ld16x2(tcol, tcol + 16u, va, vb);
                        if (c0 + 32 >= col_hi) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&acc_empty[half]);
                        }
                        cp_async_wait<1>();  // this pass's copies have landed (the next pass's may still be in flight)
                        __syncwarp();
                        const int live = col_hi - c0;
                        const TX *xs_ = reinterpret_cast<const TX *>(buf + s * seg) + jj;  // token tt: + tt * 32 elements
                        const float *ivs = reinterpret_cast<const float *>(buf + 128 * 32) + s;
                        // First every token's term of this lane's stream, in place of its accumulator (shared-memory reads and
                        // arithmetic only: a store to u in between would fence the next token's reads behind it, both being
                        // generic addresses).  Then the four streams of a column - lanes l, l ^ 1, l ^ 2, l ^ 3 - are added
                        // four tokens at a time by a reduce-scatter: three shuffles instead of the eight of four butterflies,
                        // and it leaves each of the four lanes with the sum of one token, which that lane stores.
#pragma unroll
                        for (int t = 0; t < 16; ++t) {
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                const int tt = t + 16 * hf;
                                const float z = hf ? vb[t] : va[t];
                                const float c = __fdividef(load_as_f32(xs_, tt * 32) * ivs[tt * 4] * nwp, 1.0f + __expf(-z));
                                if (hf) vb[t] = c;
                                else va[t] = c;
                            }
                        }
                        const bool b0 = (lane & 1) != 0, b1 = (lane & 2) != 0;
                        const int mine = (b0 ? 2 : 0) + (b1 ? 1 : 0);  // which of a group's four tokens this lane ends up with
                        TX *up = static_cast<TX *>(hc.u) + (int64_t)(it.start + c0 + mine) * hc.d + j;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float ta = i < 4 ? va[4 * i] : vb[4 * i - 16], tb = i < 4 ? va[4 * i + 1] : vb[4 * i - 15];
                            const float tc = i < 4 ? va[4 * i + 2] : vb[4 * i - 14], td = i < 4 ? va[4 * i + 3] : vb[4 * i - 13];
                            // lanes with bit 0 clear keep tokens a, b and send c, d; the others the reverse
                            const float k0 = (b0 ? tc : ta) + __shfl_xor_sync(0xffffffffu, b0 ? ta : tc, 1);
                            const float k1 = (b0 ? td : tb) + __shfl_xor_sync(0xffffffffu, b0 ? tb : td, 1);
                            // lanes with bit 1 clear keep the first of the two and send the second; the others the reverse
                            const float sum = (b1 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, b1 ? k0 : k1, 2);
                            if (4 * i + mine < live) store_from_f32(up, (int64_t)(4 * i) * hc.d, sum * 0.25f);
                        }
                    }
                }
                cp_async_wait<0>();
            };
            if (a.hc.f32) run(std::true_type{});
            else run(std::false_type{});
        }
    } else if (warp < kEpiWarps) {
        // ===================== epilogue =====================
        // Lane = weight row: 32 tokens at a time from tensor memory into registers (two loads of 16 columns), then one
        // store per token straight to global memory - for a fixed token a warp's rows are contiguous bytes.  Tensor
        // memory goes back to the MMA warp as soon as the item's last columns are in registers.  What depends on the
        // token - the output row of its slot, or its line in the tile-blocked h - is computed by lane t for token t of
        // the pass and handed round by shuffles.
        uint32_t acc_count = 0;
        const int64_t I = a.N / 2;
        const bool tiled_out = MODE == kTcSwiglu && a.out_f16 >= 3;
        const bool h_as_f16 = a.out_f16 != 0, q4_order = a.out_f16 == 2 || a.out_f16 == 3;
        const int quad = warp & 3;                         // the lane quadrant this warp may read
        const int col_lo = (warp >> 2) * (kTile / kEpiSets);  // this warp's set takes the columns [col_lo, col_lo + kTile / kEpiSets)
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int up_lane = lane >> 4;  // SwiGLU: lanes 16-31 hold the up rows of the h columns of lanes 0-15
        for (int item = blockIdx.x; item < n_items && !*abort_v; item += gridDim.x) {
            const Item it = item_info<TILE>(a, item, rbs);
            const bool valid = it.bucket < a.E;
            // per-thread constants of the item: byte offset of this thread's element inside a token's output row / line
            int64_t elem_off;
            uint32_t xor_chunk = 0;  // tile-blocked h: 16-byte chunk of the line, before the per-token swizzle
            bool row_ok;
            if (MODE == kTcSwiglu) {
                const int64_t j = (int64_t)it.rb * (kRows / 2) + quad * 16 + (lane & 15);  // h column
                const int j7 = (int)(j & 7), pos = q4_order ? (((j7 & 3) << 1) | (j7 >> 2)) : j7;  // [0 4 1 5 2 6 3 7]
                row_ok = j < I;
                if (tiled_out) elem_off = (j >> 6) * a.L.S * 128 + pos * 2, xor_chunk = (uint32_t)((j & 63) >> 3);
                else elem_off = ((j & ~(int64_t)7) + pos) * 2;
            } else {
                const int64_t r = (int64_t)it.rb * kRows + quad * 32 + lane;
                row_ok = r < a.N;
                elem_off = r * (MODE == kTcPartial ? 4 : 2);
            }
            // Slot of token n of the item (fetched one pass ahead; nothing may depend on the loaded value before the next
            // pass, or the in-order issue would stall this pass's stores behind it).
            auto token_slot = [&](int n) -> int { return (tiled_out || n >= it.cnt) ? 0 : slot_at(it.start + n); };
            // Offset of a token's output row / line, in 16-byte units.
            auto token_off = [&](int n, int slot) -> uint32_t {
                if (tiled_out) return (uint32_t)(it.start + n) * 8u;
                return (uint32_t)(((int64_t)slot * (MODE == kTcSwiglu ? I * 2 : a.N * (MODE == kTcPartial ? 4 : 2))) >> 4);
            };
            const int col_hi = min(it.cnt, col_lo + kTile / kEpiSets);  // this set's tokens: [col_lo, col_hi)
            int slot_nxt = token_slot(col_lo + lane);
            uint32_t half = 0;
            if (valid) {
                half = acc_count % kAccs;
                const uint32_t acc_phase = (acc_count / kAccs) & 1u;
                ++acc_count;
                if (lane == 0 && !mbar_wait(&acc_full[half], acc_phase, abort_v, a.wait_limit_ns)) raise_abort(item, 4);
                __syncwarp();
                if (*abort_v) break;
                tc_fence_after();
                if (col_lo >= col_hi && lane == 0) mbar_arrive(&acc_empty[half]);  // none of the item's tokens are this set's
            }
            unsigned char *out = static_cast<unsigned char *>(a.out) + elem_off;
            for (int c0 = col_lo; c0 < col_hi; c0 += 32) {
                float va[16], vb[16];  // this row's accumulators of tokens c0 .. c0 + 15 and c0 + 16 .. c0 + 31
                if (valid) {
                    const uint32_t col = lane_addr + half * (uint32_t)kTile + (uint32_t)c0;
                    tc_ld16x2(col, col + 16u, va, vb);
                    if (c0 + 32 >= col_hi) {  // this set's last columns are out: its share of the accumulator is free
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[half]);
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 16; ++t) va[t] = vb[t] = qnan_f32();
                }
                const uint32_t off_cur = token_off(c0 + lane, slot_nxt);
                if (c0 + 32 < col_hi) slot_nxt = token_slot(c0 + 32 + lane);
                const int live = it.cnt - c0;  // tokens of this pass; the columns past them are computed and dropped
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    if (MODE == kTcSwiglu) {
                        // the gate lane finishes token c0 + t, its up lane token c0 + 16 + t: each sends the other the
                        // value that one needs (kernels/moe_grouped.hip:508-524: from the FP32 accumulators, rounded once)
                        const float mine = up_lane ? va[t] : vb[t], theirs = __shfl_xor_sync(0xffffffffu, mine, 16);
                        const float g = up_lane ? theirs : va[t], u = up_lane ? vb[t] : theirs;
                        // a token's line of the tile-blocked h follows from its position; otherwise its slot's row was
                        // looked up by lane (t or t + 16) of this pass
                        const int64_t off = tiled_out ? (int64_t)(it.start + c0 + t + 16 * up_lane) << 7
                                                      : (int64_t)__shfl_sync(0xffffffffu, off_cur, t + (lane & 16)) << 4;
                        const uint16_t b = __bfloat16_as_ushort(__float2bfloat16_rn(silu_fast(g) * u));
                        const uint16_t hv = h_as_f16 ? __half_as_ushort(__float2half_rn(bf16_bits_to_f32(b))) : b;
                        const uint32_t sw = tiled_out ? ((xor_chunk ^ (uint32_t)(t & 7)) << 4) : 0u;
                        if (row_ok && t + 16 * up_lane < live) *reinterpret_cast<uint16_t *>(out + off + sw) = hv;
                    } else {
                        const int64_t off_a = (int64_t)__shfl_sync(0xffffffffu, off_cur, t) << 4;
                        const int64_t off_b = (int64_t)__shfl_sync(0xffffffffu, off_cur, t + 16) << 4;
                        if (MODE == kTcPartial) {
                            if (row_ok && t < live) *reinterpret_cast<float *>(out + off_a) = va[t];
                            if (row_ok && t + 16 < live) *reinterpret_cast<float *>(out + off_b) = vb[t];
                        } else {  // BF16 rows: the plain gather's y, or the per-slot dots as kernels/moe_grouped.hip:47-57 stores them
                            if (row_ok && t < live) *reinterpret_cast<uint16_t *>(out + off_a) = __bfloat16_as_ushort(__float2bfloat16_rn(va[t]));
                            if (row_ok && t + 16 < live) *reinterpret_cast<uint16_t *>(out + off_b) = __bfloat16_as_ushort(__float2bfloat16_rn(vb[t]));
                        }
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
        if (warp == kBCopyWarp && lane == 0)
            for (const unsigned long long t0 = global_ns(); global_ns() - t0 < 50000ull;) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

// Two boxes of 64 bytes x 64 rows fill a ring slot; 16-byte chunks swizzled in the 64-byte mode so that the producers'
// 16-byte reads of consecutive rows hit every bank once.
template <int BITS, int MODE>
int launch_tiled_tc(const char *fn, TcArgs a, int64_t G, cudaStream_t st) {
    SXB_CHECK(a.x_kind == 3, fn, ": the tiled tcgen05 kernel takes tile-blocked activations only");
    CUtensorMap wmap;
    if (int rc = tensor_map_2d(fn, a.q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)(BITS == 4 ? a.K / 2 : a.K), (uint64_t)(a.E * a.N),
                               (uint64_t)(BITS == 4 ? a.K / 2 : a.K), 64u, (uint32_t)(kRows / 2), CU_TENSOR_MAP_SWIZZLE_64B, &wmap))
        return rc;
    // A long contraction (gate/up: d = 4096 is 64 k-blocks) takes the wider tile; a short one (down: I = 1024 is 16 k-blocks)
    // the narrower, double-buffered one: there the epilogue weighs as much as the mainloop.
    // (the up mix of the hyper-connections contracts over its rank, at most 1024: it has the narrower form only)
    const bool wide = MODE != kTcHcUp && a.K >= 2048;
    using SB = Shape<kTcTileB>;
    using SA = Shape<kTcTileA, MODE == kTcHcUp>;
    const size_t smem = (wide ? (size_t)SB::kStages * SB::kStageBytes + (size_t)SB::kWSlots * kWSlotBytes
                              : (size_t)SA::kStages * SA::kStageBytes + (size_t)SA::kWSlots * kWSlotBytes) + 1024 +
                        (MODE == kTcHcUp ? (size_t)SA::kEpiWarps * 2 * kHcUpBufBytes : 0);
    auto go = [&](auto kern) -> int {
        SXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn, ": reserving shared memory");
        kern<<<(unsigned)sm_count(), wide ? SB::kThreads : SA::kThreads, smem, st>>>(a, wmap);
        return SXB_OK;
    };
    if constexpr (MODE != kTcHcUp) {
        if (wide) {
            switch (G) {
                case 32: return go(tiled_tc_kernel<BITS, 32, MODE, kTcTileB>);
                case 64: return go(tiled_tc_kernel<BITS, 64, MODE, kTcTileB>);
                default: return go(tiled_tc_kernel<BITS, 128, MODE, kTcTileB>);
            }
        }
    }
    switch (G) {
        case 32: return go(tiled_tc_kernel<BITS, 32, MODE, kTcTileA>);
        case 64: return go(tiled_tc_kernel<BITS, 64, MODE, kTcTileA>);
        default: return go(tiled_tc_kernel<BITS, 128, MODE, kTcTileA>);
    }
}

template int launch_tiled_tc<4, kTcGather>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<4, kTcSwiglu>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<4, kTcPartial>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<4, kTcPartialBf16>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<8, kTcGather>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<8, kTcSwiglu>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<8, kTcPartial>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<8, kTcPartialBf16>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<4, kTcHcUp>(const char *, TcArgs, int64_t, cudaStream_t);
template int launch_tiled_tc<8, kTcHcUp>(const char *, TcArgs, int64_t, cudaStream_t);

}  // namespace sxb
