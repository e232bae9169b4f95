// One token of the MoE router, by one warp: top-k of the token's E logits (larger first, a tie to the lower index), the
// softmax over the picks, the optional shared slot.  Shared by the router kernel (router.cu) and the one-CTA
// router + pack kernel of small batches (route_pack.cu).  Arithmetic: kernels/moe_router.hip:82-111.
#pragma once

#include "common.cuh"

#include <climits>

namespace sxb {

constexpr int kRouterLanes = 32;

// Order-preserving map float -> uint32 (finite values and infinities): a < b  <=>  key(a) < key(b).
// -0 is folded onto +0 first, so the two compare equal as they do as floats.
__device__ inline uint32_t order_key(float v) {
    const uint32_t u = __float_as_uint(v + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// row: the token's logits; id_row / coef_row: its A output slots.  The whole warp calls this (lane = its lane).
template <typename T, int NV>
__device__ inline void route_token(const T *__restrict__ row, int lane, int64_t m, int E, int k, const T *__restrict__ shared,
                                   int64_t shared_ld, int32_t shared_id, int32_t *__restrict__ id_row,
                                   float *__restrict__ coef_row, int A, uint32_t *err) {
    constexpr int kLanes = kRouterLanes;
    uint32_t key[NV];
    float val[NV];
    int bad = INT_MAX;  // smallest index of a non-finite logit (E = the shared gate)
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int e = lane + j * kLanes;
        const float x = e < E ? load_as_f32(row, e) : -INFINITY;
        val[j] = x;
        key[j] = e < E ? order_key(x) : 0u;  // 0 sorts below every real key (key(-inf) = 0x007fffff)
        if (e < E && !isfinite(x)) bad = min(bad, e);
    }
    float sl = 0.f;
    if (shared != nullptr) {
        sl = load_as_f32(shared, m * shared_ld);
        if (!isfinite(sl)) bad = min(bad, E);
    }
    bad = __reduce_min_sync(0xffffffffu, bad);
    if (bad != INT_MAX) {
        if (lane == 0) raise_error(err, (uint32_t)m, (uint32_t)bad);
        for (int a = lane; a < A; a += kLanes) {
            id_row[a] = -1;
            coef_row[a] = qnan_f32();
        }
        return;
    }

    // This lane's best: ascending scan with a strict > keeps the lower index on a tie.
    uint32_t lk;
    int li, lj;
    auto lane_best = [&] {
        lk = 0u, li = INT_MAX, lj = -1;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (key[j] > lk) lk = key[j], li = lane + j * kLanes, lj = j;
    };
    lane_best();
    float my_v = 0.f, top = 0.f;
    int my_i = -1;
    for (int r = 0; r < k; ++r) {
        const uint32_t best_key = __reduce_max_sync(0xffffffffu, lk);
        const int best_i = __reduce_min_sync(0xffffffffu, lk == best_key ? li : INT_MAX);
        const int owner = best_i % kLanes;
        float bv = 0.f;
        if (lane == owner) {
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (j == lj) bv = val[j], key[j] = 0u;  // static register indices only
            lane_best();
        }
        bv = __shfl_sync(0xffffffffu, bv, owner);
        if (r == 0) top = bv;
        if (lane == r) my_v = bv, my_i = best_i;
    }

    // Softmax over the k picks; the sum is the reference's 32-lane xor butterfly, so equal exps give equal sums.
    const float ex = lane < k ? expf(my_v - top) : 0.f;
    float sum = ex;
#pragma unroll
    for (int off = kLanes / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane < k) {
        id_row[lane] = my_i;
        coef_row[lane] = ex / sum;
    }
    if (shared != nullptr && lane == 0) {
        id_row[k] = shared_id;
        coef_row[k] = 1.0f / (1.0f + expf(-sl));
    }
}

}  // namespace sxb
