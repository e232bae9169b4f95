// Layout of the grouping workspace shared by the pack (route_pack.cu) and the expert kernels that walk it.
#pragma once

#include "common.cuh"

namespace sxb {

constexpr int64_t kMoeMaxExperts = 1023;   // E + 1 buckets fit one 1024-thread CTA (kernels/moe_grouped.hpp:43)
constexpr int64_t kMoeMaxSlots = 1 << 20;  // kernels/moe_grouped.hpp:44
constexpr int kSegSlots = 1024;            // slots one warp places in the multi-CTA pack
// Tokens per work item of the tcgen05 kernel for tile-blocked activations (multiples of 16): the narrower tile has two
// accumulators in tensor memory (short contractions, where an item's epilogue must run under the next item's mainloop),
// the wider one has one (long contractions, where sharing a dequantization between more tokens pays more).
constexpr int kTcTileA = 192, kTcTileB = 256;

// Word (int32) offsets into the workspace.
//   header [8]: n_tiles8, S, E, n_tiles128, ep_mode, 0, 0, 0
//   offsets [E + 2]: bucket b's slots are slots[offsets[b] .. offsets[b + 1]); bucket E = invalid ids (or, in
//                    expert-parallel mode, every slot that is not this rank's); offsets[E + 1] = S
//   slots [S]: slot index s = m * A + a, ascending inside a bucket
//   t8_bucket / t8_start [T8max]: tiles of up to 8 slots (the streaming kernels); t128_*: up to 128 (tcgen05)
//   segbad [nseg], scratch [nseg][E + 1]: the multi-CTA pack's per-segment first invalid slot and histograms
//   tta [1 + 2 * TtAmax], ttb [1 + 2 * TtBmax]: a count, then bucket / start of tiles of up to kTcTileA and kTcTileB slots
//                    (the tcgen05 kernel for tile-blocked activations: a work item is 128 weight rows x one such tile)
struct RouteWords {
    int64_t S, E, T8max, T128max, TtAmax, TtBmax, nseg;
    int64_t offsets, slots, t8_bucket, t8_start, t128_bucket, t128_start, segbad, scratch, tta_n, tta_bucket, tta_start, ttb_n, ttb_bucket, ttb_start, total;
};
RouteWords route_words(int64_t M, int64_t A, int64_t E);
// The workspace (route_words(M * E, 1, E)) of the grouping in which slot m * E + b belongs to bucket b, for all m < M: what
// sxb_moe_group_routes writes for ids[m * E + b] = b, without the ids or the sort.
int regular_routes(const char *fn, int64_t M, int64_t E, void *ws, size_t ws_bytes, sxb_stream_t stream);

}  // namespace sxb
