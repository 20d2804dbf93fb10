// Shared host/device helpers for the oxq kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/oxq.h"

#define OXQ_EXPORT extern "C" __attribute__((visibility("default")))

namespace oxq {

// ---- host-side error plumbing -------------------------------------------
// Records a printf-style message for oxq_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);
void clear_error();

#define OXQ_REQUIRE(cond, code, ...)                      \
    do {                                                  \
        if (!(cond)) return ::oxq::fail((code), __VA_ARGS__); \
    } while (0)

#define OXQ_CUDA(expr)                                                                          \
    do {                                                                                        \
        cudaError_t e__ = (expr);                                                               \
        if (e__ != cudaSuccess)                                                                 \
            return ::oxq::fail(OXQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));   \
    } while (0)

// Launch-error check that leaves asynchronous errors to the caller's sync.
#define OXQ_LAUNCH_CHECK(name)                                                                      \
    do {                                                                                            \
        cudaError_t e__ = cudaGetLastError();                                                       \
        if (e__ != cudaSuccess)                                                                     \
            return ::oxq::fail(OXQ_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

// Experiment knobs: environment variables are looked at only in builds made with -DOXQ_TUNING
// (passed through OXQ_NVCC_FLAGS); the shipped library never reads the environment.
#ifdef OXQ_TUNING
inline const char *tuning_env(const char *name) { return getenv(name); }
#else
inline const char *tuning_env(const char *) { return nullptr; }
#endif

// Streaming multiprocessors of the current device (cached per device; 148 on B200).
inline int sm_count()
{
    static int count[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (count[device] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) v = 148;
        count[device] = v;
    }
    return count[device];
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline bool valid_dtype(int d) { return d == OXQ_F32 || d == OXQ_F16 || d == OXQ_BF16; }
inline size_t dtype_size(int d) { return d == OXQ_F32 ? 4 : 2; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- device helpers --------------------------------------------------------
#ifdef __CUDACC__

// Scalar load of an f32/f16/bf16 element widened to f32 (exact).
__device__ __forceinline__ float load_as_f32(const void *p, int dtype, size_t idx)
{
    if (dtype == OXQ_F32) return reinterpret_cast<const float *>(p)[idx];
    if (dtype == OXQ_F16) return __half2float(reinterpret_cast<const __half *>(p)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[idx]);
}

// Store with one round-to-nearest-even narrowing (none for f32).
template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void store_as(void *p, int dtype, size_t idx, float v)
{
    if (dtype == OXQ_F32) reinterpret_cast<float *>(p)[idx] = v;
    else if (dtype == OXQ_F16) reinterpret_cast<__half *>(p)[idx] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16 *>(p)[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float half_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// E4M3fn byte -> f32, every encoding exact: 1-4-3, bias 7, e=0 subnormal
// m * 2^-9, S.1111.111 NaN, no infinities.
__device__ __forceinline__ float e4m3_to_f32(uint32_t v)
{
    uint32_t s = (v & 0x80u) << 24, e = (v >> 3) & 0xFu, m = v & 7u;
    if (e == 0) return __uint_as_float(s | __float_as_uint((float)m * 0.001953125f));
    if (e == 15 && m == 7) return __uint_as_float(s | 0x7FC00000u);
    return __uint_as_float(s | ((e + 120u) << 23) | (m << 20));
}

// E2M1 code (bit 3 = sign) -> f32: {0, .5, 1, 1.5, 2, 3, 4, 6}.
__device__ __forceinline__ float e2m1_to_f32(uint32_t c)
{
    uint32_t mag = c & 7u;
    // 0 -> 0, 1 -> 0.5; otherwise exponent (mag >> 1) - 1 with one mantissa bit.
    float v = mag < 2 ? 0.5f * (float)mag : __uint_as_float(((126u + (mag >> 1)) << 23) | ((mag & 1u) << 22));
    return (c & 8u) ? -v : v;
}

// E8M0 exponent byte -> 2^(s-127); 0xFF is NaN, 0 is the subnormal 2^-127.
__device__ __forceinline__ float e8m0_to_f32(uint32_t s)
{
    if (s == 0xFFu) return __uint_as_float(0x7FC00000u);
    if (s == 0u) return __uint_as_float(0x00400000u);
    return __uint_as_float(s << 23);
}

// Two bf16 (one 32-bit word, element 0 in the low half) and two more -> f16 pairs (lo0, lo1) of each
// word, saturated to the largest finite f16 (the conversion rounds to nearest even; every bf16
// inside the f16 normal range converts exactly).
__device__ __forceinline__ uint32_t f32x2_to_f16x2_sat(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16_lo_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

#endif // __CUDACC__

// ---- programmatic dependent launch --------------------------------------------------------------
// A decode kernel spends a good part of its few microseconds starting up and draining. Launched with
// allow_early_start(), a kernel may become resident while the previous kernel on the stream is still
// running; it calls pdl_launch_dependents() at entry (so that its own successor may do the same) and
// pdl_wait() before it touches anything a previous kernel may write or still read (x, y, routing
// tables). Only reads of weights, scales and zero points, which no kernel writes, go in front of
// the wait. pdl_wait() returns when the previous kernel has completed and its writes are visible;
// without the launch attribute both calls do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif
inline void allow_early_start(cudaLaunchAttribute *attrs, unsigned int &count)
{
    if (const char *env = tuning_env("OXQ_PDL"))
        if (env[0] == '0') return;
    attrs[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[count].val.programmaticStreamSerializationAllowed = 1;
    count += 1;
}

} // namespace oxq
