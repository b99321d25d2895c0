// Shared device/host helpers for the dynb kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dynb.h"

namespace dynb {

// ---- small vector type usable for float and double records -----------------------------
template <typename T> struct Vec4;
template <> struct __align__(16) Vec4<float> { float x, y, z, w; };
template <> struct __align__(32) Vec4<double> { double x, y, z, w; };

template <typename T> struct IntOf;
template <> struct IntOf<float> { using type = int32_t; };
template <> struct IntOf<double> { using type = int64_t; };

__device__ __forceinline__ float bits_to_real(int32_t v, float) { return __int_as_float(v); }
__device__ __forceinline__ double bits_to_real(int32_t v, double) { return __longlong_as_double((long long)v); }
__device__ __forceinline__ int32_t real_to_bits(float v) { return __float_as_int(v); }
__device__ __forceinline__ int32_t real_to_bits(double v) { return (int32_t)__double_as_longlong(v); }

// ---- order-preserving float <-> unsigned maps for atomicMin / atomicMax ----------------
__device__ __forceinline__ uint32_t ordered_u32(float f)
{
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unordered_f32(uint32_t u)
{
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}
__device__ __forceinline__ unsigned long long ordered_u64(double f)
{
    unsigned long long u = (unsigned long long)__double_as_longlong(f);
    return (u & 0x8000000000000000ull) ? ~u : (u | 0x8000000000000000ull);
}
__device__ __forceinline__ double unordered_f64(unsigned long long u)
{
    return __longlong_as_double((long long)((u & 0x8000000000000000ull) ? (u & 0x7fffffffffffffffull) : ~u));
}

// ---- warp primitives ---------------------------------------------------------------------
__device__ __forceinline__ int warp_excl_scan(int v, int lane, int* total)
{
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    *total = __shfl_sync(0xffffffffu, x, 31);
    return x - v;
}

__device__ __forceinline__ uint32_t lanemask_lt()
{
    uint32_t m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// ---- host-side launch check --------------------------------------------------------------
#define DYNB_CUDA_OK(expr)                                \
    do {                                                  \
        cudaError_t _e = (expr);                          \
        if (_e != cudaSuccess) return dynb::fail_cuda(_e, #expr); \
    } while (0)

int fail_cuda(cudaError_t e, const char* what);
int fail_arg(const char* what);
void set_last_error(const char* msg);

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
static inline int sm_count_cached()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace dynb
