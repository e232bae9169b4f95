// Writes the golden strixw file of tests/golden with the REFERENCE's own writer and quantizers (formats/strixw.cpp,
// formats/q4.cpp, formats/q8.cpp compiled where they lie by oracle/Makefile), and reads it back with the reference's own
// reader.  TEST INFRASTRUCTURE: it pins this repository's strixw reader and its test-side writer to the reference's bytes.
//
//   strixw_golden <out.strixw>
// Contents (a miniature MoE layer, E = 3 experts, d = 64, I = 32): deterministic weights w[i] = ((i * 2654435761 >> 8 & 0xffff)
// / 65536 - 0.5) * 0.1, quantized by quantize_q4 / quantize_q8;
//   layers.0.mlp.experts_gate_up  Q4 G64 [(E + 1) * 2I, d], experts = E + 1 (the shared expert stacked last), three parts
//   layers.0.mlp.experts_down     Q8 G32 [E * d, I], experts = E
//   layers.0.mlp.router           F32 [E + 1, d]
//   norm                          BF16 [d]
#include "formats/q4.hpp"
#include "formats/q8.hpp"
#include "formats/strixw.hpp"

#include <cstdint>
#include <cstdio>
#include <vector>

static std::vector<float> pattern(size_t n, uint32_t salt) {
    std::vector<float> v(n);
    for (size_t i = 0; i < n; ++i) {
        const uint32_t h = ((uint32_t)(i + salt) * 2654435761u) >> 8 & 0xffffu;
        v[i] = ((float)h / 65536.0f - 0.5f) * 0.1f;
    }
    return v;
}

int main(int argc, char **argv) {
    if (argc != 2) return 1;
    using namespace strix;
    const int64_t E = 3, d = 64, I = 32;
    try {
        std::vector<StrixwTensor> plan(4);
        plan[0].name = "layers.0.mlp.experts_gate_up", plan[0].encoding = StrixwEncoding::Q4RowMajor;
        plan[0].shape = {(E + 1) * 2 * I, d}, plan[0].group_size = 64, plan[0].experts = E + 1;
        plan[0].parts = {{"layers.0.mlp.experts.gate_up_proj", 0, E * 2 * I},
                         {"layers.0.mlp.shared_expert.gate_proj.weight", E * 2 * I, I},
                         {"layers.0.mlp.shared_expert.up_proj.weight", E * 2 * I + I, I}};
        plan[1].name = "layers.0.mlp.experts_down", plan[1].encoding = StrixwEncoding::Q8RowMajor;
        plan[1].shape = {E * d, I}, plan[1].group_size = 32, plan[1].experts = E;
        plan[2].name = "layers.0.mlp.router", plan[2].encoding = StrixwEncoding::F32, plan[2].shape = {E + 1, d};
        plan[3].name = "norm", plan[3].encoding = StrixwEncoding::BF16, plan[3].shape = {d};
        StrixwWriter w(argv[1], {{"arch", "qwen4_exp"}, {"made_by", "the reference's StrixwWriter"}}, plan);
        const std::vector<float> gu = pattern((size_t)((E + 1) * 2 * I * d), 1), dn = pattern((size_t)(E * d * I), 2);
        const Q4Weight q4 = quantize_q4(gu.data(), (E + 1) * 2 * I, d, 64);
        w.write(0, StrixwRole::Q, q4.q.data(), q4.q.size());
        w.write(0, StrixwRole::Scale, q4.scale.data(), q4.scale.size() * 2);
        w.write(0, StrixwRole::Min, q4.minv.data(), q4.minv.size() * 2);
        const Q8Weight q8 = quantize_q8(dn.data(), E * d, I, 32);
        w.write(1, StrixwRole::Q, q8.q.data(), q8.q.size());
        w.write(1, StrixwRole::Scale, q8.scale.data(), q8.scale.size() * 2);
        w.write(1, StrixwRole::Min, q8.minv.data(), q8.minv.size() * 2);
        const std::vector<float> router = pattern((size_t)((E + 1) * d), 3);
        w.write(2, StrixwRole::Data, router.data(), router.size() * 4);
        std::vector<uint16_t> norm((size_t)d);
        for (int64_t i = 0; i < d; ++i) norm[(size_t)i] = (uint16_t)(0x3f80 + i);  // BF16 bits near 1.0
        w.write(3, StrixwRole::Data, norm.data(), norm.size() * 2);
        w.finish();
        StrixwFile f(argv[1]);  // the reference's reader accepts what its writer wrote
        f.verify_hashes(2);
        std::printf("%s: %llu bytes, %zu tensors, data at %llu\n", argv[1], (unsigned long long)f.file_bytes(), f.tensors().size(),
                    (unsigned long long)f.data_offset());
    } catch (const std::exception &e) {
        std::fprintf(stderr, "%s\n", e.what());
        return 2;
    }
    return 0;
}
