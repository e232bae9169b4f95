// Pack: groups the S = M*A routed slots by expert (a counting sort) and cuts every expert's run of slots into the
// tiles the expert kernels iterate over.  C ABI twin of moe_group_routes / moe_route_workspace_bytes
// (kernels/moe_grouped.hpp:48-54; the reference's kernel is kernels/moe_grouped.hip:136-188, one 1024-thread block
// whose order inside a bucket is whatever its LDS atomics give).
//
// Here the sort is stable - inside a bucket, slots ascend - so the whole workspace is a pure function of ids and can
// be compared word for word with a CPU counting sort.  Ranks inside a bucket come from `match.any` warp votes, never
// from the arrival order of atomics.
//   S <= kSmallSlots: one CTA does everything (decode: S = 160 is five warp rounds).
//   larger S: three launches - per-warp-segment histograms, one CTA that scans them into bucket offsets / per-segment
//   bases / tile lists, and a scatter in which every warp places its own segment in order.

#include "route_pack.cuh"

#include <algorithm>
#include "router_token.cuh"

namespace sxb {
namespace {

constexpr int kPackThreads = 1024;
constexpr int kSmallSlots = 2048;
constexpr int kSegWarps = 8;  // warps (segments) per CTA in the histogram / scatter launches

__device__ inline int bucket_of(int32_t id, int e_lo, int E_local) {
    const int b = id - e_lo;
    return (b < 0 || b >= E_local) ? E_local : b;
}

// Exclusive scan of v over the CTA's kPackThreads threads; *total = the sum.  buf: 33 ints of shared memory.
__device__ inline int cta_exclusive_scan(int v, int *buf, int *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) buf[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = buf[lane], wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += t;
        }
        buf[lane] = wi - w;
        if (lane == 31) buf[32] = wi;
    }
    __syncthreads();
    const int excl = incl - v + buf[warp];
    *total = buf[32];
    __syncthreads();
    return excl;
}

// Writes offsets, the header and the four tile lists from per-bucket counts (thread b owns bucket b).
// tile_first: 4 * 1025 ints of shared memory.
__device__ void emit_layout(int count, const RouteWords &L, int32_t *ws, int *scanbuf, int *tile_first, bool ep) {
    const int b = threadIdx.x, E = (int)L.E;
    const bool owner = b <= E;
    // Tiles are cut for buckets 0..E-1, and for the overflow bucket E only outside expert-parallel mode (there its
    // slots are invalid ids whose outputs must become NaN; in EP mode they belong to other ranks and are skipped).
    const bool tiled = owner && (b < E || !ep);
    int total_slots, n8, n128, nta, ntb;
    const int start = cta_exclusive_scan(owner ? count : 0, scanbuf, &total_slots);
    const int t8 = tiled ? (count + 7) / 8 : 0, t128 = tiled ? (count + 127) / 128 : 0;
    const int first8 = cta_exclusive_scan(t8, scanbuf, &n8);
    const int first128 = cta_exclusive_scan(t128, scanbuf, &n128);
    const int firstta = cta_exclusive_scan(tiled ? (count + kTcTileA - 1) / kTcTileA : 0, scanbuf, &nta);
    const int firsttb = cta_exclusive_scan(tiled ? (count + kTcTileB - 1) / kTcTileB : 0, scanbuf, &ntb);
    int32_t *offsets = ws + L.offsets;
    if (owner) offsets[b] = start;
    if (b <= E + 1) {  // first tile of each bucket; entry E + 1 = the total
        tile_first[b] = b <= E ? first8 : n8;
        tile_first[1025 + b] = b <= E ? first128 : n128;
        tile_first[2050 + b] = b <= E ? firstta : nta;
        tile_first[3075 + b] = b <= E ? firsttb : ntb;
    }
    if (b == 0) {
        offsets[E + 1] = total_slots;
        ws[0] = n8, ws[1] = (int32_t)L.S, ws[2] = E, ws[3] = n128, ws[4] = ep ? 1 : 0, ws[5] = 0, ws[6] = 0, ws[7] = 0;
        ws[L.tta_n] = nta, ws[L.ttb_n] = ntb;
    }
    __syncthreads();
    // Tiles in parallel: tile t belongs to the last bucket whose first tile is <= t.
    for (int pass = 0; pass < 4; ++pass) {
        const int *first = tile_first + pass * 1025;
        const int n = pass == 0 ? n8 : pass == 1 ? n128 : pass == 2 ? nta : ntb;
        const int rows = pass == 0 ? 8 : pass == 1 ? 128 : pass == 2 ? kTcTileA : kTcTileB;
        int32_t *tb = ws + (pass == 0 ? L.t8_bucket : pass == 1 ? L.t128_bucket : pass == 2 ? L.tta_bucket : L.ttb_bucket);
        int32_t *ts = ws + (pass == 0 ? L.t8_start : pass == 1 ? L.t128_start : pass == 2 ? L.tta_start : L.ttb_start);
        for (int t = threadIdx.x; t < n; t += kPackThreads) {
            int lo = 0, hi = E + 1;  // invariant: first[lo] <= t < first[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (first[mid] <= t) lo = mid;
                else hi = mid;
            }
            // lo is the last bucket whose first tile is <= t; empty buckets (first[b] == first[b + 1]) never win
            tb[t] = lo;
            ts[t] = offsets[lo] + (t - first[lo]) * rows;
        }
    }
}

// One warp places the slots [s0, s1) in order: rank inside a round from match.any, bucket cursors in shared memory.
__device__ inline void warp_place(const int32_t *ids, int s0, int s1, int e_lo, int E_local, int *cursor, int32_t *slots) {
    const int lane = threadIdx.x & 31;
    for (int base = s0; base < s1; base += 32) {
        const int s = base + lane;
        const bool live = s < s1;
        const int b = live ? bucket_of(ids[s], e_lo, E_local) : -1 - lane;  // dead lanes match nobody
        const unsigned peers = __match_any_sync(0xffffffffu, b);
        if (live) {
            const int rank = __popc(peers & ((1u << lane) - 1u));
            const int at = cursor[b];
            slots[at + rank] = s;
            __syncwarp(peers);
            if (rank == 0) cursor[b] = at + __popc(peers);
        }
        __syncwarp();
    }
}

// The whole pack of a small batch by one CTA of kPackThreads threads.
__device__ void pack_small_body(const int32_t *__restrict__ ids, const RouteWords &L, int E_total, int e_lo, bool ep, int32_t *ws,
                                uint32_t *err) {
    __shared__ int cnt[kPackThreads], scanbuf[33], tile_first[4 * 1025];
    __shared__ int first_bad;
    const int t = threadIdx.x, S = (int)L.S, E = (int)L.E;
    cnt[t] = 0;
    if (t == 0) first_bad = 0x7fffffff;
    __syncthreads();
    for (int s = t; s < S; s += kPackThreads) {
        const int32_t id = ids[s];
        atomicAdd(&cnt[bucket_of(id, e_lo, E)], 1);  // counts do not depend on the order of arrival
        if (id < 0 || id >= E_total) atomicMin(&first_bad, s);
    }
    __syncthreads();
    if (t == 0 && first_bad != 0x7fffffff) raise_error(err, (uint32_t)ids[first_bad], (uint32_t)first_bad);
    const int count = t <= E ? cnt[t] : 0;
    emit_layout(count, L, ws, scanbuf, tile_first, ep);
    __syncthreads();
    if (t <= E) cnt[t] = ws[L.offsets + t];  // cnt becomes the bucket cursors
    __syncthreads();
    if (t < 32) warp_place(ids, 0, S, e_lo, E, cnt, ws + L.slots);
}

__global__ void __launch_bounds__(kPackThreads)
    pack_small_kernel(const int32_t *__restrict__ ids, RouteWords L, int E_total, int e_lo, bool ep, int32_t *ws,
                      uint32_t *err) {
    pack_small_body(ids, L, E_total, e_lo, ep, ws, err);
}

// Router and pack of a small batch (decode: a few dozen tokens) as ONE launch of one CTA: every warp routes tokens
// (route_token), the CTA then packs the slots it has just written.  Same words out as moe_router + moe_group_routes.
template <int NV>
__global__ void __launch_bounds__(kPackThreads)
    route_small_kernel(const float *__restrict__ logits, int64_t ld, int M, int E_total, int k, int32_t *__restrict__ ids,
                       float *__restrict__ coef, RouteWords L, int e_lo, bool ep, int32_t *ws, uint32_t *router_err,
                       uint32_t *expert_err) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int m = warp; m < M; m += kPackThreads / 32)
        route_token<float, NV>(logits + (int64_t)m * ld, lane, m, E_total, k, nullptr, 1, 0, ids + (int64_t)m * k,
                               coef + (int64_t)m * k, k, router_err);
    __threadfence_block();
    __syncthreads();  // the ids written above are read by other threads of this CTA below
    pack_small_body(ids, L, E_total, e_lo, ep, ws, expert_err);
}

// Large S, launch 1: histogram of every 1024-slot segment (one warp each) into scratch [nseg][E + 1], and the
// segment's first invalid slot into segbad [nseg].
__global__ void __launch_bounds__(32 * kSegWarps)
    pack_hist_kernel(const int32_t *__restrict__ ids, RouteWords L, int E_total, int e_lo, int32_t *ws) {
    __shared__ int hist[kSegWarps][1024];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, E = (int)L.E, S = (int)L.S;
    const int seg = blockIdx.x * kSegWarps + warp;
    if (seg >= L.nseg) return;
    for (int b = lane; b <= E; b += 32) hist[warp][b] = 0;
    __syncwarp();
    const int s0 = seg * kSegSlots, s1 = min(S, s0 + kSegSlots);
    int bad = 0x7fffffff;
    for (int s = s0 + lane; s < s1; s += 32) {
        const int32_t id = ids[s];
        atomicAdd(&hist[warp][bucket_of(id, e_lo, E)], 1);
        if (id < 0 || id >= E_total) bad = min(bad, s);
    }
    bad = __reduce_min_sync(0xffffffffu, bad);
    __syncwarp();
    int32_t *out = ws + L.scratch + (int64_t)seg * (E + 1);
    for (int b = lane; b <= E; b += 32) out[b] = hist[warp][b];
    if (lane == 0) ws[L.segbad + seg] = bad;
}

// Launch 2 (one CTA): per bucket, turn the segments' counts into their exclusive prefix (the segment's base inside
// the bucket); totals -> offsets, header, tile lists; the first invalid slot -> err.
__global__ void __launch_bounds__(kPackThreads)
    pack_scan_kernel(const int32_t *__restrict__ ids, RouteWords L, bool ep, int32_t *ws, uint32_t *err) {
    __shared__ int scanbuf[33], tile_first[4 * 1025];
    const int b = threadIdx.x, E = (int)L.E;
    int total = 0;
    if (b <= E) {
        // sixteen segments at a time: the loads of a chunk are independent of one another (a chain of dependent
        // read-modify-writes over 160 segments was most of this launch)
        int32_t *col = ws + L.scratch + b;
        const int64_t stride = E + 1;
        for (int seg0 = 0; seg0 < L.nseg; seg0 += 16) {
            int c[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) c[i] = seg0 + i < L.nseg ? col[(int64_t)(seg0 + i) * stride] : 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (seg0 + i < L.nseg) col[(int64_t)(seg0 + i) * stride] = total;
                total += c[i];
            }
        }
    }
    int bad = 0x7fffffff;
    for (int seg = b; seg < L.nseg; seg += kPackThreads) bad = min(bad, ws[L.segbad + seg]);
    bad = __reduce_min_sync(0xffffffffu, bad);
    __shared__ int bad_w[32];
    if ((b & 31) == 0) bad_w[b >> 5] = bad;
    __syncthreads();
    if (b == 0) {
        for (int w = 1; w < 32; ++w) bad = min(bad, bad_w[w]);
        if (bad != 0x7fffffff) raise_error(err, (uint32_t)ids[bad], (uint32_t)bad);
    }
    emit_layout(total, L, ws, scanbuf, tile_first, ep);
}

// Launch 3: every warp places its segment, starting each bucket at offsets[b] + the segment's base.
__global__ void __launch_bounds__(32 * kSegWarps)
    pack_scatter_kernel(const int32_t *__restrict__ ids, RouteWords L, int e_lo, int32_t *ws) {
    __shared__ int cursor[kSegWarps][1024];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, E = (int)L.E, S = (int)L.S;
    const int seg = blockIdx.x * kSegWarps + warp;
    if (seg >= L.nseg) return;
    const int32_t *base = ws + L.scratch + (int64_t)seg * (E + 1);
    for (int b = lane; b <= E; b += 32) cursor[warp][b] = ws[L.offsets + b] + base[b];
    __syncwarp();
    const int s0 = seg * kSegSlots;
    warp_place(ids, s0, min(S, s0 + kSegSlots), e_lo, E, cursor[warp], ws + L.slots);
}

int group_routes(const char *fn, const int32_t *ids, int64_t M, int64_t A, int64_t E_total, int64_t e_lo,
                 int64_t E_local, bool ep, void *ws, size_t ws_bytes, uint32_t *err, sxb_stream_t stream) {
    SXB_CHECK(ids != nullptr && ws != nullptr && err != nullptr, fn, ": null pointer (ids=", (const void *)ids, ", ws=", ws,
              ", err=", (const void *)err, ")");
    SXB_CHECK(M >= 1 && A >= 1 && A <= 64 && E_local >= 1 && E_local <= kMoeMaxExperts && M * A <= kMoeMaxSlots, fn,
              ": M = ", M, ", A = ", A, ", E = ", E_local, " (A 1..64, E 1..", kMoeMaxExperts, ", M*A <= ", kMoeMaxSlots, ")");
    SXB_CHECK(e_lo >= 0 && e_lo + E_local <= E_total, fn, ": experts [", e_lo, ", ", e_lo + E_local, ") outside [0, ",
              E_total, ")");
    const RouteWords L = route_words(M, A, E_local);
    SXB_CHECK(ws_bytes >= (size_t)L.total * 4, fn, ": workspace of ", ws_bytes, " bytes, needs ", L.total * 4);
    SXB_CHECK(reinterpret_cast<uintptr_t>(ws) % 4 == 0, fn, ": workspace ", ws, " must be 4-byte aligned");
    auto st = static_cast<cudaStream_t>(stream);
    auto *w = static_cast<int32_t *>(ws);
    if (L.S <= kSmallSlots) {
        pack_small_kernel<<<1, kPackThreads, 0, st>>>(ids, L, (int)E_total, (int)e_lo, ep, w, err);
    } else {
        const unsigned ctas = (unsigned)((L.nseg + kSegWarps - 1) / kSegWarps);
        pack_hist_kernel<<<ctas, 32 * kSegWarps, 0, st>>>(ids, L, (int)E_total, (int)e_lo, w);
        pack_scan_kernel<<<1, kPackThreads, 0, st>>>(ids, L, ep, w, err);
        pack_scatter_kernel<<<ctas, 32 * kSegWarps, 0, st>>>(ids, L, (int)e_lo, w);
    }
    SXB_CHECK_LAUNCH(fn, " M=", M, " A=", A, " E=", E_local);
    return SXB_OK;
}

// The workspace of a regular grouping, written without ids: S = M * E slots, slot m * E + b in bucket b for every m, so that
// bucket b holds M slots in ascending order.  CTA 0 writes offsets, header and tile lists; every CTA writes slots.
__global__ void __launch_bounds__(kPackThreads) regular_routes_kernel(RouteWords L, int per_bucket, int32_t *ws) {
    __shared__ int scanbuf[33], tile_first[4 * 1025];
    const int E = (int)L.E;
    int32_t *slots = ws + L.slots;
    for (int64_t pos = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; pos < L.S; pos += (int64_t)gridDim.x * blockDim.x)
        slots[pos] = (int32_t)((pos % per_bucket) * E + pos / per_bucket);
    if (blockIdx.x == 0) emit_layout((int)threadIdx.x < E ? per_bucket : 0, L, ws, scanbuf, tile_first, false);
}

}  // namespace

int regular_routes(const char *fn, int64_t M, int64_t E, void *ws, size_t ws_bytes, sxb_stream_t stream) {
    SXB_CHECK(ws != nullptr && M >= 1 && E >= 1 && E <= kMoeMaxExperts && M * E <= kMoeMaxSlots, fn, ": M = ", M, ", E = ", E, ", ws = ", ws);
    const RouteWords L = route_words(M * E, 1, E);
    SXB_CHECK(ws_bytes >= (size_t)L.total * 4 && reinterpret_cast<uintptr_t>(ws) % 4 == 0, fn, ": workspace of ", ws_bytes, " bytes, needs ", L.total * 4);
    const unsigned ctas = (unsigned)std::min<int64_t>((L.S + kPackThreads - 1) / kPackThreads, (int64_t)sm_count() * 2);
    regular_routes_kernel<<<ctas, kPackThreads, 0, static_cast<cudaStream_t>(stream)>>>(L, (int)M, static_cast<int32_t *>(ws));
    SXB_CHECK_LAUNCH(fn, " regular grouping M=", M, " E=", E);
    return SXB_OK;
}

RouteWords route_words(int64_t M, int64_t A, int64_t E) {
    RouteWords L;
    L.S = M * A, L.E = E;
    L.T8max = L.S / 8 + E + 2, L.T128max = L.S / 128 + E + 2;
    L.nseg = L.S <= kSmallSlots ? 0 : (L.S + kSegSlots - 1) / kSegSlots;
    L.offsets = 8;
    L.slots = L.offsets + E + 2;
    L.t8_bucket = L.slots + L.S;
    L.t8_start = L.t8_bucket + L.T8max;
    L.t128_bucket = L.t8_start + L.T8max;
    L.t128_start = L.t128_bucket + L.T128max;
    L.segbad = L.t128_start + L.T128max;
    L.scratch = L.segbad + L.nseg;
    L.TtAmax = L.S / kTcTileA + E + 2, L.TtBmax = L.S / kTcTileB + E + 2;
    L.tta_n = L.scratch + L.nseg * (E + 1);
    L.tta_bucket = L.tta_n + 1;
    L.tta_start = L.tta_bucket + L.TtAmax;
    L.ttb_n = L.tta_start + L.TtAmax;
    L.ttb_bucket = L.ttb_n + 1;
    L.ttb_start = L.ttb_bucket + L.TtBmax;
    L.total = L.ttb_start + L.TtBmax;
    return L;
}

}  // namespace sxb

using namespace sxb;

namespace sxb {
// {2, work item, role}: the record of a device-side wait of the tcgen05 kernels that ran out (grouped_tc.cu).
int tc_status_error(const char *what, const uint32_t e[3]) {
    static const char *roles[] = {"an unknown role",
                                  "a weight producer waiting for a free operand stage",
                                  "an MMA warp waiting for free accumulators",
                                  "an MMA warp waiting for a filled operand stage",
                                  "the epilogue waiting for the accumulators",
                                  "the activation copy thread waiting for a free operand stage",
                                  "the weight-code copy thread waiting for a free ring slot",
                                  "a weight producer waiting for its packed codes"};
    last_error() = cat(what ? what : "", ": a tcgen05 kernel gave up a wait at work item ", e[1], " (",
                       roles[e[2] >= 1 && e[2] <= 7 ? e[2] : 0], "); its outputs are incomplete");
    return SXB_ERR_DATA;
}
}  // namespace sxb

extern "C" {

size_t sxb_moe_route_workspace_bytes(int64_t M, int64_t A, int64_t E) {
    if (!(M >= 1 && A >= 1 && E >= 1 && E <= kMoeMaxExperts && M * A <= kMoeMaxSlots)) {
        fail_check(SXB_FILE_, __LINE__, __func__, "M >= 1 && A >= 1 && 1 <= E <= 1023 && M * A <= 2^20",
                   cat("moe_route_workspace_bytes: M = ", M, ", A = ", A, ", E = ", E));
        return 0;
    }
    return (size_t)route_words(M, A, E).total * 4;
}

int sxb_route_layout(int64_t M, int64_t A, int64_t E, int64_t out[8]) {
    SXB_CHECK(out != nullptr && M >= 1 && A >= 1 && E >= 1 && E <= kMoeMaxExperts && M * A <= kMoeMaxSlots,
              "route_layout: M = ", M, ", A = ", A, ", E = ", E);
    const RouteWords L = route_words(M, A, E);
    out[0] = 0, out[1] = L.offsets, out[2] = L.slots, out[3] = L.t8_bucket, out[4] = L.t8_start, out[5] = L.t128_bucket,
    out[6] = L.t128_start, out[7] = L.total;
    return SXB_OK;
}

int sxb_check_grouped_status(const void *ws, const char *what) {
    SXB_CHECK(ws != nullptr, "check_grouped_status(", what, "): null workspace");
    int32_t head[8];
    SXB_CUDA(cudaMemcpy(head, ws, sizeof(head), cudaMemcpyDeviceToHost), "reading the workspace header for ", what);
    if (head[5] == 0) return SXB_OK;
    const uint32_t e[3] = {(uint32_t)head[5], (uint32_t)head[6], (uint32_t)head[7]};
    return tc_status_error(what, e);
}

int sxb_moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, void *ws, size_t ws_bytes, uint32_t *err,
                         sxb_stream_t stream) {
    return group_routes("moe_group_routes", ids, M, A, E, 0, E, false, ws, ws_bytes, err, stream);
}

int sxb_moe_group_routes_ep(const int32_t *ids, int64_t M, int64_t A, int64_t E_total, int64_t e_lo, int64_t E_local,
                            void *ws, size_t ws_bytes, uint32_t *err, sxb_stream_t stream) {
    return group_routes("moe_group_routes_ep", ids, M, A, E_total, e_lo, E_local, true, ws, ws_bytes, err, stream);
}

int sxb_moe_route_small(const float *logits, int64_t ld, int64_t M, int64_t E_total, int64_t k, int64_t e_lo, int64_t E_local,
                        int32_t *ids, float *coef, void *ws, size_t ws_bytes, uint32_t *router_err, uint32_t *expert_err,
                        sxb_stream_t stream) {
    const char *fn = "moe_route_small";
    SXB_CHECK(logits != nullptr && ids != nullptr && coef != nullptr && ws != nullptr && router_err != nullptr && expert_err != nullptr,
              fn, ": null pointer");
    SXB_CHECK(E_total >= 1 && E_total <= 1024 && k >= 1 && k <= E_total && k <= 32 && ld >= E_total, fn, ": E = ", E_total, ", k = ", k,
              ", ld = ", ld, " (E 1..1024, k 1..min(E, 32), ld >= E)");
    SXB_CHECK(M >= 1 && M * k <= kSmallSlots, fn, ": M * k = ", M * k, " slots, this one-CTA form takes at most ", kSmallSlots,
              " (use moe_router + moe_group_routes)");
    SXB_CHECK(E_local >= 1 && E_local <= kMoeMaxExperts && e_lo >= 0 && e_lo + E_local <= E_total, fn, ": experts [", e_lo, ", ",
              e_lo + E_local, ") outside [0, ", E_total, ")");
    const bool ep = E_local != E_total;
    const RouteWords L = route_words(M, k, E_local);
    SXB_CHECK(ws_bytes >= (size_t)L.total * 4, fn, ": workspace of ", ws_bytes, " bytes, needs ", L.total * 4);
    auto st = static_cast<cudaStream_t>(stream);
    auto *w = static_cast<int32_t *>(ws);
#define SXB_ROUTE_SMALL(NV) \
    route_small_kernel<NV><<<1, kPackThreads, 0, st>>>(logits, ld, (int)M, (int)E_total, (int)k, ids, coef, L, (int)e_lo, ep, w, router_err, expert_err)
    if (E_total <= 128) SXB_ROUTE_SMALL(4);
    else if (E_total <= 256) SXB_ROUTE_SMALL(8);
    else if (E_total <= 512) SXB_ROUTE_SMALL(16);
    else SXB_ROUTE_SMALL(32);
#undef SXB_ROUTE_SMALL
    SXB_CHECK_LAUNCH(fn, " M=", M, " E=", E_total, " k=", k);
    return SXB_OK;
}

}  // extern "C"
