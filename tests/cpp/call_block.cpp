// A C++ host that drives the MoE block through strix_b200_shim.hpp exactly as the reference's forward does
// (runtime/qwen4exp.cpp:3156-3196: moe_router, moe_group_routes, the grouped SwiGLU gather, the grouped combine), linked
// against libstrix_b200.so.  The test harness writes the inputs to a file, runs this program and compares the output file
// bit for bit with what the Python launcher sequence computed from the same inputs.
//
//   call_block <in> <out>
//   in : int64 header {M, E, A, d, I, G_gu, G_dn}, then x [M, d] BF16, logits [M, E] FP32,
//        gate_up {q [E*2I, d/2], scale, min [E*2I, d/G]}, down {q [E*d, I/2], scale, min [E*d, I/G]}   (Q4 both)
//   out: ids [M, A] int32, coef [M, A] FP32, y [M, d] BF16
#include "strix_b200_shim.hpp"

#include <cstdio>
#include <cstdlib>
#include <vector>

namespace sk = strix::kernels;

#define CUDA_OK(call)                                                                   \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) {                                                        \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));            \
            return 2;                                                                   \
        }                                                                               \
    } while (0)

template <typename T>
static cudaError_t dmalloc(T **p, size_t bytes) { return cudaMalloc(reinterpret_cast<void **>(p), bytes); }

template <typename T>
static T *upload(std::FILE *f, size_t count) {
    std::vector<T> host(count);
    if (std::fread(host.data(), sizeof(T), count, f) != count) {
        std::fprintf(stderr, "short read\n");
        std::exit(3);
    }
    T *dev = nullptr;
    if (dmalloc(&dev, count * sizeof(T)) != cudaSuccess) std::exit(4);
    if (cudaMemcpy(dev, host.data(), count * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) std::exit(5);
    return dev;
}

int main(int argc, char **argv) {
    if (argc != 3) return 1;
    std::FILE *f = std::fopen(argv[1], "rb");
    if (!f) return 1;
    int64_t hd[7];
    if (std::fread(hd, sizeof(int64_t), 7, f) != 7) return 1;
    const int64_t M = hd[0], E = hd[1], A = hd[2], d = hd[3], I = hd[4], Ggu = hd[5], Gdn = hd[6];
    uint16_t *x = upload<uint16_t>(f, M * d);
    float *logits = upload<float>(f, M * E);
    strix::Q4DeviceView gu, dn;
    gu.q = upload<uint8_t>(f, E * 2 * I * d / 2), gu.scale = upload<uint16_t>(f, E * 2 * I * d / Ggu);
    gu.minv = upload<uint16_t>(f, E * 2 * I * d / Ggu), gu.N = E * 2 * I, gu.K = d, gu.G = Ggu;
    dn.q = upload<uint8_t>(f, E * d * I / 2), dn.scale = upload<uint16_t>(f, E * d * I / Gdn);
    dn.minv = upload<uint16_t>(f, E * d * I / Gdn), dn.N = E * d, dn.K = I, dn.G = Gdn;
    std::fclose(f);

    cudaStream_t stream;
    CUDA_OK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    int32_t *ids;
    float *coef, *partial;
    uint16_t *h, *y;
    uint32_t *err;
    void *ws;
    size_t ws_bytes = 0;
    try {
        ws_bytes = sk::moe_route_workspace_bytes(M, A, E);
        CUDA_OK(dmalloc(&ids, M * A * 4));
        CUDA_OK(dmalloc(&coef, M * A * 4));
        CUDA_OK(dmalloc(&ws, ws_bytes));
        CUDA_OK(dmalloc(&h, M * A * I * 2));
        CUDA_OK(dmalloc(&partial, M * A * d * 4));
        CUDA_OK(dmalloc(&y, M * d * 2));
        CUDA_OK(dmalloc(&err, 8 * 4));
        CUDA_OK(cudaMemset(err, 0, 8 * 4));
        // the call block of the reference's forward, launcher by launcher
        sk::moe_router(logits, E, M, E, A, nullptr, 1, 0, ids, coef, sk::Act::F32, err, stream);
        sk::moe_group_routes(ids, M, A, E, ws, ws_bytes, err + 4, stream);
        sk::linear_q4_experts_gather_grouped_swiglu(x, gu, E, ws, ws_bytes, M, A, h, sk::Act::BF16, sk::MoeMath::F32, stream);
        sk::linear_q4_experts_combine_grouped(h, dn, E, ids, coef, ws, ws_bytes, partial, M, A, y, sk::Act::BF16, sk::MoeMath::F32,
                                              stream);
        CUDA_OK(cudaStreamSynchronize(stream));
        sk::check_router_error(err, "call_block");
        sk::check_expert_error(err + 4, "call_block");
        // a refused call surfaces as strix::Error with the library's message
        bool threw = false;
        try {
            sk::moe_router(logits, E - 1, M, E, A, nullptr, 1, 0, ids, coef, sk::Act::F32, err, stream);
        } catch (const strix::Error &e) {
            threw = std::string(e.what()).find("ld") != std::string::npos;
        }
        if (!threw) {
            std::fprintf(stderr, "a bad ld was not refused\n");
            return 6;
        }
    } catch (const strix::Error &e) {
        std::fprintf(stderr, "strix::Error: %s\n", e.what());
        return 7;
    }
    std::vector<int32_t> ids_h(M * A);
    std::vector<float> coef_h(M * A);
    std::vector<uint16_t> y_h(M * d);
    CUDA_OK(cudaMemcpy(ids_h.data(), ids, M * A * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(coef_h.data(), coef, M * A * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(y_h.data(), y, M * d * 2, cudaMemcpyDeviceToHost));
    std::FILE *o = std::fopen(argv[2], "wb");
    if (!o) return 1;
    std::fwrite(ids_h.data(), 4, ids_h.size(), o);
    std::fwrite(coef_h.data(), 4, coef_h.size(), o);
    std::fwrite(y_h.data(), 2, y_h.size(), o);
    std::fclose(o);
    return 0;
}
