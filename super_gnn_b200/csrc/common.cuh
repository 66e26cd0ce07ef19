// Shared host/device helpers for the sm_100a kernels of supergnn_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/supergnn_b200.h"

#define SGNN_API __attribute__((visibility("default")))

namespace sgnn {

// ---- host side: status and error text -------------------------------------
void set_error(const char *fmt, ...);  // records the text for sgnn_last_error_string()

#define SGNN_REQUIRE(cond, code, ...)          \
    do {                                       \
        if (!(cond)) {                         \
            ::sgnn::set_error(__VA_ARGS__);    \
            return (code);                     \
        }                                      \
    } while (0)

#define SGNN_CUDA_OK(expr)                                                              \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess) {                                                        \
            ::sgnn::set_error("%s failed: %s", #expr, cudaGetErrorString(_e));          \
            return SGNN_ERR_CUDA;                                                       \
        }                                                                               \
    } while (0)

// Launch check: catches configuration errors without synchronising.
#define SGNN_LAUNCH_OK(what)                                                            \
    do {                                                                                \
        cudaError_t _e = cudaPeekAtLastError();                                         \
        if (_e != cudaSuccess) {                                                        \
            ::sgnn::set_error("launch of %s failed: %s", what, cudaGetErrorString(_e)); \
            return SGNN_ERR_CUDA;                                                       \
        }                                                                               \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// SM count of the current device (cached per device).
int sm_count();

// ---- device side ----------------------------------------------------------
#ifdef __CUDACC__

constexpr unsigned FULL = 0xffffffffu;

// Streaming (read-once) loads: keep them out of L1 so the gathered rows keep it.
__device__ __forceinline__ int ld_stream(const int *p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }

// fp32 reduction into global memory, 16 bytes at a time (sm_90+).
__device__ __forceinline__ void red_add_v4(float *addr, float4 v)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
                 "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void red_add(float *addr, float v) { atomicAdd(addr, v); }

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

// fp32 -> bf16 bits, round to nearest even (NaN stays NaN).
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f)
{
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// Largest r in [0, n) with a[r] <= target, for a non-decreasing a with a[0] <= target.
// Whole-warp 32-ary search: every step probes 32 evenly spaced entries at once, so the
// dependent-load chain is ceil(log32 n) long instead of log2 n.
__device__ __forceinline__ int64_t warp_upper_row(const int64_t *__restrict__ a, int64_t n, int64_t target, int lane)
{
    int64_t lo = 0, hi = n;  // invariant: a[lo] <= target, answer in [lo, hi)
    while (hi - lo > 1) {
        const int64_t span = hi - lo;
        const int64_t step = (span + 31) / 32;
        const int64_t idx = lo + (int64_t)lane * step;
        const bool ok = (idx < hi) && (__ldg(a + idx) <= target);
        const unsigned m = __ballot_sync(FULL, ok);  // bit 0 always set (a[lo] <= target); set bits are a prefix
        const int last = 31 - __clz(m);
        const int64_t nlo = lo + (int64_t)last * step;
        int64_t nhi = nlo + step;
        if (nhi > hi) nhi = hi;
        lo = nlo;
        hi = nhi;
    }
    return lo;
}

#endif  // __CUDACC__
}  // namespace sgnn
