// Shared host/device helpers for libreflex_b200: status plumbing, dtype traits,
// per-op rounding arithmetic that reproduces torch's eager CPU sequence.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/reflex_b200.h"

namespace rfx {

// ---- host-side status plumbing ------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);
// Returns RFX_SUCCESS when the current device is compute capability 10.x.
int check_device();
int sm_count();
int check_launch(const char* what);

// Debug switches: the comma-separated words of the environment variable REFLEX_B200_DEBUG, read once
// (std::call_once), or whatever rfx_debug_set_flags() put in their place. One atomic word; nothing
// else in the library looks at the environment.
enum : uint32_t {
    kDbgNoTensorCore = 1u,    // "no_tc": the scalar kernels instead of the tcgen05 ones (attention, linear + norm)
    kDbgPrefillNoSplit = 2u,  // "prefill_nosplit": chunked prefill streams whole contexts per CTA
    kDbgMixedOn = 4u,         // "mixed=1": one-row requests of a split batch always go to the decode kernel
    kDbgMixedOff = 8u,        // "mixed=0": never
    kDbgTma2d = 16u,          // "tma2d": the decode kernel's 2-D tensor maps (one copy per 128-byte half)
};
uint32_t debug_flags();

// "Done once per device" marks (an opt-in attribute set, a cached query). Atomic, so that host threads
// may race to do the work twice but never see a torn value.
struct PerDeviceOnce {
    std::atomic<int> v[64];
    bool done(int dev) const { return dev >= 0 && dev < 64 && v[dev].load(std::memory_order_acquire) != 0; }
    void mark(int dev, int value = 1) { if (dev >= 0 && dev < 64) v[dev].store(value, std::memory_order_release); }
    int value(int dev) const { return (dev >= 0 && dev < 64) ? v[dev].load(std::memory_order_acquire) : 0; }
};

#define RFX_REQUIRE(cond, ...)                                   \
    do {                                                         \
        if (!(cond)) return ::rfx::fail(RFX_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

inline cudaStream_t as_stream(rfx_stream s) { return reinterpret_cast<cudaStream_t>(s); }

inline size_t dtype_size(int dt) { return dt == RFX_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == RFX_F32 || dt == RFX_BF16 || dt == RFX_F16; }

template <typename T> __host__ __device__ inline T ceil_div(T a, T b) { return (a + b - 1) / b; }
template <typename T> __host__ __device__ inline T round_up(T a, T b) { return ceil_div(a, b) * b; }

// ---- device-side dtype traits ---------------------------------------------------
template <typename T> struct Num;
template <> struct Num<float> {
    __device__ static float to_f(float v) { return v; }
    __device__ static float from_f(float v) { return v; }
};
template <> struct Num<__nv_bfloat16> {
    __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Num<int8_t> {  // int8 KV pool: the stored integer; its scale is applied by the caller
    __device__ static float to_f(int8_t v) { return (float)v; }
};
template <> struct Num<__half> {
    __device__ static float to_f(__half v) { return __half2float(v); }
    __device__ static __half from_f(float v) { return __float2half_rn(v); }
};

// One torch-eager elementwise op: operands widened to fp32, one IEEE op with
// round-to-nearest (no FMA contraction), result rounded to T. For 16-bit T this is what
// torch's CPU kernels do per op; for fp32 it is the op itself.
template <typename T> __device__ inline T mul_r(T a, T b) {
    return Num<T>::from_f(__fmul_rn(Num<T>::to_f(a), Num<T>::to_f(b)));
}
template <typename T> __device__ inline T sub_r(T a, T b) {
    return Num<T>::from_f(__fsub_rn(Num<T>::to_f(a), Num<T>::to_f(b)));
}
template <typename T> __device__ inline T add_r(T a, T b) {
    return Num<T>::from_f(__fadd_rn(Num<T>::to_f(a), Num<T>::to_f(b)));
}

// Two 16-bit values side by side. The product of two bf16 (or fp16) numbers is exact in fp32, so
// "widen, multiply in fp32, round to T" is one rounding of the exact product, which is what the
// packed multiply does for both lanes in one instruction (results below the fp32 normal range, where
// the fp32 product itself would already have rounded, are the one place the two could differ).
// Sums are not exact in fp32, so add_r / sub_r keep the widened form.
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
    using P = __nv_bfloat162;
    __device__ static P mul(P a, P b) { return __hmul2(a, b); }
    __device__ static float2 widen(P a) { return __bfloat1622float2(a); }
    __device__ static P round(float a, float b) { return __floats2bfloat162_rn(a, b); }
    __device__ static P both_low(P a) { return __low2bfloat162(a); }
};
template <> struct Pair16<__half> {
    using P = __half2;
    __device__ static P mul(P a, P b) { return __hmul2(a, b); }
    __device__ static float2 widen(P a) { return __half22float2(a); }
    __device__ static P round(float a, float b) { return __floats2half2_rn(a, b); }
    __device__ static P both_low(P a) { return __low2half2(a); }
};

// The RoPE pair rotation of kernels/rope/triton_rope.py:230-240 in torch-eager rounding:
//   y1 = x1*c - x2*s ; y2 = x1*s + x2*c, each op rounded to T.
template <typename T>
__device__ inline void rope_pair(T x1, T x2, T c, T s, T& y1, T& y2) {
    y1 = sub_r<T>(mul_r<T>(x1, c), mul_r<T>(x2, s));
    y2 = add_r<T>(mul_r<T>(x1, s), mul_r<T>(x2, c));
}

__device__ inline float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Dispatch a lambda-like macro over the three dtypes.
#define RFX_DISPATCH_DTYPE(dt, T, ...)                         \
    do {                                                       \
        if ((dt) == RFX_F32) { using T = float; __VA_ARGS__; } \
        else if ((dt) == RFX_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else { using T = __half; __VA_ARGS__; }                \
    } while (0)

}  // namespace rfx
