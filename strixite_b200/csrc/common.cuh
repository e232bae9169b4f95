// Shared host/device helpers of the sm_100a MoE library: BF16 bit conversions, the error-message plumbing behind
// the C ABI's return codes, argument checks common to several launchers.
#pragma once

#include "strix_b200.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <sstream>
#include <string>

namespace sxb {

// ---- error plumbing -------------------------------------------------------------------------------------------
// The reference throws strix::Error with "func (file:line): check `cond` failed: message" (common/check.hpp:59-62).
// A C ABI cannot throw: the message goes to a thread-local string, the code to the caller.
std::string &last_error();

template <typename... Args>
std::string cat(Args &&...args) {
    std::ostringstream os;
    (os << ... << args);
    return os.str();
}

int fail_check(const char *file, int line, const char *func, const char *cond, const std::string &msg);
int fail_cuda(const char *file, int line, const char *func, cudaError_t e, const std::string &msg);

#define SXB_FILE_ (__builtin_strrchr(__FILE__, '/') ? __builtin_strrchr(__FILE__, '/') + 1 : __FILE__)

#define SXB_CHECK(cond, ...)                                                                             \
    do {                                                                                                 \
        if (!(cond)) return ::sxb::fail_check(SXB_FILE_, __LINE__, __func__, #cond, ::sxb::cat(__VA_ARGS__)); \
    } while (0)

// After a launch: cudaGetLastError, the reference's STRIX_HIP_CHECK_LAUNCH (common/hip_check.hpp:50).
#define SXB_CHECK_LAUNCH(...)                                                                            \
    do {                                                                                                 \
        cudaError_t e_ = cudaGetLastError();                                                             \
        if (e_ != cudaSuccess) return ::sxb::fail_cuda(SXB_FILE_, __LINE__, __func__, e_, ::sxb::cat(__VA_ARGS__)); \
    } while (0)

#define SXB_CUDA(call, ...)                                                                              \
    do {                                                                                                 \
        cudaError_t e_ = (call);                                                                         \
        if (e_ != cudaSuccess) return ::sxb::fail_cuda(SXB_FILE_, __LINE__, __func__, e_, ::sxb::cat(__VA_ARGS__)); \
    } while (0)

inline const char *act_name(int act) { return act == SXB_ACT_F32 ? "F32" : act == SXB_ACT_BF16 ? "BF16" : "?"; }
inline bool act_ok(int act) { return act == SXB_ACT_F32 || act == SXB_ACT_BF16; }
inline int64_t act_bytes(int act) { return act == SXB_ACT_F32 ? 4 : 2; }

inline bool apart(const void *a, int64_t an, const void *b, int64_t bn) {
    const auto ab = reinterpret_cast<uintptr_t>(a), bb = reinterpret_cast<uintptr_t>(b);
    return ab + (uintptr_t)an <= bb || bb + (uintptr_t)bn <= ab;
}
inline bool aligned16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

// ---- device helpers ---------------------------------------------------------------------------------------------
__host__ __device__ inline float bf16_bits_to_f32(uint16_t b) {
#ifdef __CUDA_ARCH__
    return __uint_as_float((uint32_t)b << 16);
#else
    uint32_t u = (uint32_t)b << 16;
    float f;
    __builtin_memcpy(&f, &u, 4);
    return f;
#endif
}
// Round to nearest even; Inf stays Inf, NaN stays a (quiet) NaN - the reference's conversion (common/bf16.hpp:21-27).
__host__ __device__ inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
#ifdef __CUDA_ARCH__
    u = __float_as_uint(f);
#else
    __builtin_memcpy(&u, &f, 4);
#endif
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x0040u : 0u));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ inline float as_stored_bf16(float v) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }
__device__ inline float qnan_f32() { return __int_as_float(0x7fc00000); }
// kernels/swiglu.hip:22
__device__ inline float silu_f32(float v) { return v / (1.0f + expf(-v)); }

// First writer wins (kernels/linear_q4.hip:166-173).
__device__ inline void raise_error(uint32_t *err, uint32_t a, uint32_t b) {
    if (atomicCAS(&err[0], 0u, 1u) == 0u) {
        err[1] = a;
        err[2] = b;
    }
}

template <typename T> __device__ inline float load_as_f32(const T *p, int64_t i);
template <> __device__ inline float load_as_f32<float>(const float *p, int64_t i) { return p[i]; }
template <> __device__ inline float load_as_f32<uint16_t>(const uint16_t *p, int64_t i) { return bf16_bits_to_f32(p[i]); }
template <> __device__ inline float load_as_f32<__half>(const __half *p, int64_t i) { return __half2float(p[i]); }
template <typename T> __device__ inline void store_from_f32(T *p, int64_t i, float v);
template <> __device__ inline void store_from_f32<float>(float *p, int64_t i, float v) { p[i] = v; }
template <> __device__ inline void store_from_f32<uint16_t>(uint16_t *p, int64_t i, float v) { p[i] = f32_to_bf16_bits(v); }
template <typename T> __device__ inline float as_stored(float v);
template <> __device__ inline float as_stored<float>(float v) { return v; }
template <> __device__ inline float as_stored<uint16_t>(float v) { return as_stored_bf16(v); }

}  // namespace sxb
