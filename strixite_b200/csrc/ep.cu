// Expert-parallel MoE layer for a C++ host: one process per GPU, rank r of N holds experts [r E / N, (r + 1) E / N) of
// every layer and owns the token rows [r T / N, (r + 1) T / N).  No counterpart in the reference, which drives one GPU.
//
//   sxb_moe_layer_ep, per layer, on the caller's stream (plus one library stream for the activation gather):
//     1. all-gather of the rank's activation rows [t, d] -> [T, d] (NCCL, on the side stream, under the routing)
//     2. router on the rank's own rows (the caller's FP32 logits), all-gather of ids and coef -> [T, A]
//     3. sxb_moe_layer on all T rows with this rank's experts: pack restricted to them, gate/up + SwiGLU, down, combine
//     4. the way back, one of
//          reduce-scatter: the rank's partial rows [T, d] FP32 -> ncclReduceScatter (sum) -> its own rows
//          peer stores:    the combine writes every row, as this rank's piece, straight into the row owner's receive
//                          buffer [N][t][d] (FP32 or F16) through peer-mapped pointers - plain stores, nothing
//                          multicast, no copy engine; a one-word NCCL all-reduce then tells every rank that all pieces
//                          have landed, and the owner adds its N pieces in rank order (FP32, deterministic)
//   The caller adds the residual (sxb_residual_add) or whatever follows.
//
// NCCL is not linked: libnccl.so.2 is opened at the first call (the copy a PyTorch process has already loaded, or the
// system's), so the rest of the library loads on hosts without it.  sxb_ep_create allocates the rank's exchange buffers
// once (device memory, cudaMalloc) and maps the peers' receive buffers (CUDA IPC); the per-layer call allocates nothing.
// There is no device-side waiting in this file: ranks meet in NCCL collectives only.

#include "experts.cuh"

#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <vector>

namespace sxb {
namespace {

// The few NCCL entry points used, by their published C signatures (nccl.h): ncclUniqueId is 128 opaque bytes passed by
// value, ncclComm_t an opaque pointer, results are ints (0 = success).
struct NcclId {
    char internal[128];
};
using NcclComm = void *;
enum { kNcclInt32 = 2, kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclUint8 = 1, kNcclSum = 0 };
struct Nccl {
    int (*GetUniqueId)(NcclId *);
    int (*CommInitRank)(NcclComm *, int, NcclId, int);
    int (*CommDestroy)(NcclComm);
    int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
    int (*ReduceScatter)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t);
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t);
    int (*GroupStart)();
    int (*GroupEnd)();
    const char *(*GetErrorString)(int);
    bool ok = false;
};

Nccl &nccl() {
    static Nccl n = [] {
        Nccl r{};
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return r;
        auto sym = [&](const char *name) { return dlsym(h, name); };
        r.GetUniqueId = reinterpret_cast<decltype(r.GetUniqueId)>(sym("ncclGetUniqueId"));
        r.CommInitRank = reinterpret_cast<decltype(r.CommInitRank)>(sym("ncclCommInitRank"));
        r.CommDestroy = reinterpret_cast<decltype(r.CommDestroy)>(sym("ncclCommDestroy"));
        r.AllGather = reinterpret_cast<decltype(r.AllGather)>(sym("ncclAllGather"));
        r.ReduceScatter = reinterpret_cast<decltype(r.ReduceScatter)>(sym("ncclReduceScatter"));
        r.AllReduce = reinterpret_cast<decltype(r.AllReduce)>(sym("ncclAllReduce"));
        r.GroupStart = reinterpret_cast<decltype(r.GroupStart)>(sym("ncclGroupStart"));
        r.GroupEnd = reinterpret_cast<decltype(r.GroupEnd)>(sym("ncclGroupEnd"));
        r.GetErrorString = reinterpret_cast<decltype(r.GetErrorString)>(sym("ncclGetErrorString"));
        r.ok = r.GetUniqueId && r.CommInitRank && r.CommDestroy && r.AllGather && r.ReduceScatter && r.AllReduce && r.GroupStart &&
               r.GroupEnd && r.GetErrorString;
        return r;
    }();
    return n;
}

#define SXB_NCCL(call, ...)                                                                                               \
    do {                                                                                                                  \
        const int r_ = (call);                                                                                            \
        if (r_ != 0) {                                                                                                    \
            last_error() = cat(__func__, " (", SXB_FILE_, ":", __LINE__, "): NCCL error ", r_, " (", nccl().GetErrorString(r_), ") ", \
                               cat(__VA_ARGS__));                                                                         \
            return SXB_ERR_CUDA;                                                                                          \
        }                                                                                                                 \
    } while (0)

constexpr int kMaxRanks = 8;
constexpr int kTimedLayers = 64;
constexpr int kMarks = 6;  // start, routes gathered, activations gathered, experts issued, pieces out, rows summed

}  // namespace
}  // namespace sxb

struct SxbEp {
    int world = 1, rank = 0, return_path = 0;
    int64_t T = 0, t = 0, d = 0, A = 0;
    sxb::NcclComm comm = nullptr;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_x = nullptr;
    uint16_t *x_all = nullptr;      // [T, d] BF16: every rank's activation rows
    int32_t *ids_loc = nullptr;     // [t, A]
    float *coef_loc = nullptr;      // [t, A]
    float *y_part = nullptr;        // [T, d] FP32 (reduce-scatter path)
    void *recv = nullptr;           // [world][t][d] pieces (peer-store paths)
    void *peer_recv[sxb::kMaxRanks] = {};
    int32_t *flag = nullptr;        // the one word of the "all pieces landed" all-reduce
    // optional phase timing: events of the last kTimedLayers calls
    bool timing = false;
    int calls = 0;
    cudaEvent_t marks[sxb::kTimedLayers][sxb::kMarks] = {};
};

namespace sxb {
namespace {

// out[m, n] = sum over ranks r, in rank order, of this rank's received pieces [world][t][N] (FP32 or F16) -> FP32 or BF16.
template <typename TP, typename TOUT>
__global__ void __launch_bounds__(256) sum_pieces_kernel(const TP *__restrict__ recv, int world, int64_t per_rank, TOUT *__restrict__ out) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= per_rank) return;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += load_as_f32(recv, (int64_t)r * per_rank + i + j);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) store_from_f32(out, i + j, v[j]);
}

void mark(SxbEp *ep, int which, cudaStream_t st) {
    if (ep->timing) cudaEventRecord(ep->marks[ep->calls % kTimedLayers][which], st);
}

}  // namespace
}  // namespace sxb

using namespace sxb;

extern "C" {

int sxb_ep_unique_id(uint8_t id[128]) {
    SXB_CHECK(id != nullptr, "ep_unique_id: null pointer");
    SXB_CHECK(nccl().ok, "ep_unique_id: libnccl.so.2 could not be opened (", dlerror() ? dlerror() : "symbols missing", ")");
    NcclId nid;
    SXB_NCCL(nccl().GetUniqueId(&nid), "creating the communicator's id");
    std::memcpy(id, nid.internal, 128);
    return SXB_OK;
}

int sxb_ep_create(const uint8_t id[128], int world, int rank, int64_t T, int64_t d, int64_t A, int return_path, SxbEp **out) {
    const char *fn = "ep_create";
    SXB_CHECK(out != nullptr && id != nullptr, fn, ": null pointer");
    SXB_CHECK(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, fn, ": rank ", rank, " of ", world, " (1..", kMaxRanks, " ranks)");
    SXB_CHECK(T >= world && T % world == 0 && d >= 8 && d % 8 == 0 && A >= 1 && A <= 64, fn, ": T = ", T, " tokens over ", world,
              " ranks, d = ", d, ", A = ", A);
    SXB_CHECK(return_path >= 0 && return_path <= 2, fn, ": return path ", return_path, " (0 reduce-scatter, 1 FP32 peer stores, 2 F16 peer stores)");
    auto *ep = new SxbEp;
    ep->world = world, ep->rank = rank, ep->return_path = return_path, ep->T = T, ep->t = T / world, ep->d = d, ep->A = A;
    *out = ep;
    SXB_CHECK(nccl().ok, fn, ": libnccl.so.2 could not be opened");
    NcclId nid;
    std::memcpy(nid.internal, id, 128);
    SXB_NCCL(nccl().CommInitRank(&ep->comm, world, nid, rank), "rank ", rank, " of ", world);
    SXB_CUDA(cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking), fn, ": side stream");
    SXB_CUDA(cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming), fn, ": event");
    SXB_CUDA(cudaEventCreateWithFlags(&ep->ev_x, cudaEventDisableTiming), fn, ": event");
    for (auto &row : ep->marks)
        for (auto &e : row) SXB_CUDA(cudaEventCreate(&e), fn, ": timing event");
    SXB_CUDA(cudaMalloc(&ep->x_all, (size_t)T * d * 2), fn, ": ", T * d * 2, " bytes for the gathered activations");
    SXB_CUDA(cudaMalloc(&ep->ids_loc, (size_t)ep->t * A * 4), fn, ": ids");
    SXB_CUDA(cudaMalloc(&ep->coef_loc, (size_t)ep->t * A * 4), fn, ": coef");
    SXB_CUDA(cudaMalloc(&ep->flag, 256), fn, ": flag");
    SXB_CUDA(cudaMemset(ep->flag, 0, 256), fn, ": flag");
    if (return_path == 0) {
        SXB_CUDA(cudaMalloc(&ep->y_part, (size_t)T * d * 4), fn, ": ", T * d * 4, " bytes for the partial rows");
        return SXB_OK;
    }
    // receive buffer for every rank's piece of this rank's rows, and the peers' buffers mapped into this process
    const size_t piece = return_path == 2 ? 2 : 4;
    SXB_CUDA(cudaMalloc(&ep->recv, (size_t)T * d * piece), fn, ": ", T * d * piece, " bytes for the received pieces");
    cudaIpcMemHandle_t mine;
    SXB_CUDA(cudaIpcGetMemHandle(&mine, ep->recv), fn, ": exporting the receive buffer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
    uint8_t *dev_h = nullptr;
    SXB_CUDA(cudaMalloc(&dev_h, (size_t)64 * (world + 1)), fn, ": handle exchange buffer");
    SXB_CUDA(cudaMemcpy(dev_h + 64 * world, &mine, 64, cudaMemcpyHostToDevice), fn, ": handle upload");
    SXB_NCCL(nccl().AllGather(dev_h + 64 * world, dev_h, 64, kNcclUint8, ep->comm, ep->side), "exchanging IPC handles");
    SXB_CUDA(cudaStreamSynchronize(ep->side), fn, ": handle exchange");
    std::vector<cudaIpcMemHandle_t> all((size_t)world);
    SXB_CUDA(cudaMemcpy(all.data(), dev_h, (size_t)64 * world, cudaMemcpyDeviceToHost), fn, ": handle download");
    SXB_CUDA(cudaFree(dev_h), fn, ": handle exchange buffer");
    for (int r = 0; r < world; ++r) {
        if (r == rank) {
            ep->peer_recv[r] = ep->recv;
            continue;
        }
        SXB_CUDA(cudaIpcOpenMemHandle(&ep->peer_recv[r], all[(size_t)r], cudaIpcMemLazyEnablePeerAccess), fn, ": mapping rank ", r,
                 "'s receive buffer");
    }
    return SXB_OK;
}

int sxb_ep_destroy(SxbEp *ep) {
    if (ep == nullptr) return SXB_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < ep->world; ++r)
        if (r != ep->rank && ep->peer_recv[r] != nullptr) cudaIpcCloseMemHandle(ep->peer_recv[r]);
    if (ep->comm) nccl().CommDestroy(ep->comm);
    cudaFree(ep->x_all), cudaFree(ep->ids_loc), cudaFree(ep->coef_loc), cudaFree(ep->y_part), cudaFree(ep->recv), cudaFree(ep->flag);
    if (ep->side) cudaStreamDestroy(ep->side);
    if (ep->ev_fork) cudaEventDestroy(ep->ev_fork);
    if (ep->ev_x) cudaEventDestroy(ep->ev_x);
    for (auto &row : ep->marks)
        for (auto &e : row)
            if (e) cudaEventDestroy(e);
    delete ep;
    return SXB_OK;
}

int sxb_ep_set_timing(SxbEp *ep, int on) {
    SXB_CHECK(ep != nullptr, "ep_set_timing: null context");
    ep->timing = on != 0;
    ep->calls = 0;
    return SXB_OK;
}

int sxb_ep_timing(SxbEp *ep, float ms[5], int *layers) {
    SXB_CHECK(ep != nullptr && ms != nullptr && layers != nullptr, "ep_timing: null pointer");
    for (int i = 0; i < 5; ++i) ms[i] = 0.f;
    const int n = std::min(ep->calls, kTimedLayers);
    *layers = n;
    if (!ep->timing || n == 0) return SXB_OK;
    SXB_CUDA(cudaDeviceSynchronize(), "ep_timing: synchronizing");
    for (int c = 0; c < n; ++c)
        for (int i = 0; i < 5; ++i) {
            float v = 0.f;
            SXB_CUDA(cudaEventElapsedTime(&v, ep->marks[c][i], ep->marks[c][i + 1]), "ep_timing: reading events");
            ms[i] += v / n;
        }
    return SXB_OK;
}

int sxb_moe_layer_ep(SxbEp *ep, const SxbMoeLayerArgs *a, sxb_stream_t stream) {
    const char *fn = "moe_layer_ep";
    SXB_CHECK(ep != nullptr && a != nullptr, fn, ": null context or argument block");
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t t = ep->t, T = ep->T, d = ep->d, A = ep->A;
    SXB_CHECK(a->M == t, fn, ": M = ", a->M, " rows, this rank owns ", t, " of ", T);
    SXB_CHECK(a->A == A && a->gate_up != nullptr && a->gate_up->K == d, fn, ": A = ", a->A, ", d = ", a->gate_up ? a->gate_up->K : 0,
              " differ from the context's ", A, ", ", d);
    SXB_CHECK(a->E_total == a->E * ep->world && a->e_lo == a->E * ep->rank, fn, ": rank ", ep->rank, " of ", ep->world, " holds experts [",
              a->e_lo, ", ", a->e_lo + a->E, ") of ", a->E_total);
    SXB_CHECK(a->shared_gate_up == nullptr, fn, ": the shared expert is not sharded: run it on the rows' owner, outside this call");
    SXB_CHECK(a->x != nullptr && a->logits != nullptr && a->y != nullptr && a->ids != nullptr && a->coef != nullptr, fn, ": null buffer");
    SXB_CHECK(a->out_act == SXB_ACT_F32 || a->out_act == SXB_ACT_BF16, fn, ": output dtype ", a->out_act);
    Nccl &nc = nccl();

    // 1. the activation rows of every rank, on the side stream, under the routing
    mark(ep, 0, st);
    SXB_CUDA(cudaEventRecord(ep->ev_fork, st), fn, ": fork");
    SXB_CUDA(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0), fn, ": fork");
    SXB_NCCL(nc.AllGather(a->x, ep->x_all, (size_t)t * d, kNcclBfloat16, ep->comm, ep->side), "all-gather of the activations");
    SXB_CUDA(cudaEventRecord(ep->ev_x, ep->side), fn, ": join");
    // 2. routes of the rank's own rows, then everybody's
    if (int rc = sxb_moe_router(a->logits, a->logits_ld, t, a->E_total, A, nullptr, 1, 0, ep->ids_loc, ep->coef_loc, SXB_ACT_F32,
                                a->router_err, stream))
        return rc;
    SXB_NCCL(nc.GroupStart(), "group");
    SXB_NCCL(nc.AllGather(ep->ids_loc, a->ids, (size_t)t * A, kNcclInt32, ep->comm, st), "all-gather of the ids");
    SXB_NCCL(nc.AllGather(ep->coef_loc, a->coef, (size_t)t * A, kNcclFloat32, ep->comm, st), "all-gather of the coefficients");
    SXB_NCCL(nc.GroupEnd(), "group");
    mark(ep, 1, st);
    SXB_CUDA(cudaStreamWaitEvent(st, ep->ev_x, 0), fn, ": join");
    mark(ep, 2, st);

    // 3. this rank's experts on all T rows
    SxbMoeLayerArgs b = *a;
    b.M = T, b.x = ep->x_all, b.logits = nullptr, b.logits_ld = 0;
    PeerOut peer{};
    if (ep->return_path == 0) {
        b.y = ep->y_part, b.out_act = SXB_ACT_F32;
        if (int rc = moe_layer_impl(&b, stream, nullptr)) return rc;
        mark(ep, 3, st);
        // 4. reduce-scatter of the partial rows
        float *dst = a->out_act == SXB_ACT_F32 ? static_cast<float *>(a->y) : ep->y_part + (size_t)ep->rank * t * d;  // in place is allowed
        SXB_NCCL(nc.ReduceScatter(ep->y_part, dst, (size_t)t * d, kNcclFloat32, kNcclSum, ep->comm, st), "reduce-scatter of the partial rows");
        mark(ep, 4, st);
        if (a->out_act != SXB_ACT_F32) {
            const unsigned blocks = (unsigned)((t * d / 4 + 255) / 256);
            sum_pieces_kernel<float, uint16_t><<<blocks, 256, 0, st>>>(dst, 1, t * d, static_cast<uint16_t *>(a->y));
            SXB_CHECK_LAUNCH(fn, " rounding the rows");
        }
        mark(ep, 5, st);
    } else {
        for (int r = 0; r < ep->world; ++r) peer.base[r] = ep->peer_recv[r];
        peer.world = ep->world, peer.rank = ep->rank, peer.t = t, peer.f16 = ep->return_path == 2;
        b.y = nullptr, b.out_act = SXB_ACT_F32;
        if (int rc = moe_layer_impl(&b, stream, &peer)) return rc;
        mark(ep, 3, st);
        // 4. every rank has stored its pieces (stream order + the collective) before anybody reads its receive buffer
        SXB_NCCL(nc.AllReduce(ep->flag, ep->flag + 32, 1, kNcclInt32, kNcclSum, ep->comm, st), "all-reduce after the peer stores");
        mark(ep, 4, st);
        const unsigned blocks = (unsigned)((t * d / 4 + 255) / 256);
        if (peer.f16) {
            if (a->out_act == SXB_ACT_F32) sum_pieces_kernel<__half, float><<<blocks, 256, 0, st>>>((const __half *)ep->recv, ep->world, t * d, (float *)a->y);
            else sum_pieces_kernel<__half, uint16_t><<<blocks, 256, 0, st>>>((const __half *)ep->recv, ep->world, t * d, (uint16_t *)a->y);
        } else {
            if (a->out_act == SXB_ACT_F32) sum_pieces_kernel<float, float><<<blocks, 256, 0, st>>>((const float *)ep->recv, ep->world, t * d, (float *)a->y);
            else sum_pieces_kernel<float, uint16_t><<<blocks, 256, 0, st>>>((const float *)ep->recv, ep->world, t * d, (uint16_t *)a->y);
        }
        SXB_CHECK_LAUNCH(fn, " summing the pieces");
        mark(ep, 5, st);
    }
    ++ep->calls;
    return SXB_OK;
}

}  // extern "C"
