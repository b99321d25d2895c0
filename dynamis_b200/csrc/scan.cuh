// Device-wide exclusive prefix sum in two launches: tile sums, then every block adds up the sums of the
// tiles before its own (a few hundred values out of L2) and scans its tile.  A separate one-block launch
// scans the tile sums only when there are very many tiles.  No block ever waits on another block, so
// there is no spin-wait anywhere.
//
// The element count may live on the device (`n_dev`): cell grids are sized by a kernel, and
// reading the count back would cost a host synchronisation.  `n_host` is then only the upper
// bound that sizes the grid.  In-place operation (out == in) is allowed when the types match.
#pragma once

#include <cstring>

#include "common.cuh"

namespace dynb {

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

template <typename T>
__device__ __forceinline__ T block_excl_scan(T v, T* block_total, T* warp_sums /* [SCAN_THREADS/32] */)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    T base = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < SCAN_THREADS / 32; w++) {
        T s = warp_sums[w];
        if (w < warp) base += s;
        tot += s;
    }
    __syncthreads();
    *block_total = tot;
    return base + x - v;
}

// A thread's SCAN_ITEMS consecutive elements: two 16-byte loads when the elements are 4 bytes wide, the array is
// 16-byte aligned and the whole run lies inside the array; element-wise otherwise (and zero past the end).
template <typename TIn, typename TOut>
__device__ __forceinline__ void scan_load_items(const TIn* in, int64_t base, int64_t n, TOut (&v)[SCAN_ITEMS])
{
    if (sizeof(TIn) == 4 && SCAN_ITEMS == 8 && base + SCAN_ITEMS <= n && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
        const uint4 a = *reinterpret_cast<const uint4*>(in + base);
        const uint4 b = *reinterpret_cast<const uint4*>(in + base + 4);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            TIn t;
            memcpy(&t, &w[i], 4);
            v[i] = (TOut)t;
        }
    } else {
#pragma unroll
        for (int i = 0; i < SCAN_ITEMS; i++) v[i] = (base + i < n) ? (TOut)in[base + i] : (TOut)0;
    }
}

// The exclusive prefix of a thread's items, run = prefix in front of the first one: 16-byte stores under the same
// conditions as the loads above.
template <typename TOut>
__device__ __forceinline__ void scan_store_items(TOut* out, int64_t base, int64_t n, TOut run, const TOut (&v)[SCAN_ITEMS])
{
    TOut r[SCAN_ITEMS];
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++) {
        r[i] = run;
        run += v[i];
    }
    if (base + SCAN_ITEMS <= n && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (sizeof(TOut) == 4 || sizeof(TOut) == 8)) {
        constexpr int PER = 16 / (int)sizeof(TOut);
#pragma unroll
        for (int q = 0; q < SCAN_ITEMS / PER; q++) {
            uint4 w;
            memcpy(&w, &r[q * PER], 16);
            *reinterpret_cast<uint4*>(out + base + q * PER) = w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < SCAN_ITEMS; i++)
            if (base + i < n) out[base + i] = r[i];
    }
}

__device__ __forceinline__ int64_t scan_count(const uint32_t* n_dev, int64_t n_host)
{
    if (n_dev == nullptr) return n_host;
    int64_t n = (int64_t)(*n_dev);
    return n < n_host ? n : n_host;
}

template <typename TIn, typename TOut>
__device__ __forceinline__ void scan_tile_sums_body(const TIn* __restrict__ in, const uint32_t* __restrict__ n_dev, int64_t n_host,
                                                    TOut* __restrict__ sums)
{
    __shared__ TOut warp_sums[SCAN_THREADS / 32];
    const int64_t n = scan_count(n_dev, n_host);
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    TOut v[SCAN_ITEMS];
    scan_load_items<TIn, TOut>(in, base, n, v);
    TOut s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++) s += v[i];
    TOut tot;
    (void)block_excl_scan<TOut>(s, &tot, warp_sums);
    if (threadIdx.x == 0) sums[blockIdx.x] = tot;
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_tile_sums_kernel(const TIn* __restrict__ in, const uint32_t* __restrict__ n_dev, int64_t n_host,
                      TOut* __restrict__ sums)
{
    scan_tile_sums_body<TIn, TOut>(in, n_dev, n_host, sums);
}

// two arrays of the same length in one launch: blockIdx.y picks the array, sums holds 2 x tiles entries
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_tile_sums_pair_kernel(const TIn* __restrict__ in0, const TIn* __restrict__ in1, const uint32_t* __restrict__ n_dev,
                           int64_t n_host, TOut* __restrict__ sums)
{
    scan_tile_sums_body<TIn, TOut>(blockIdx.y ? in1 : in0, n_dev, n_host, sums + (size_t)blockIdx.y * gridDim.x);
}

// One block scans the tile sums in place (exclusive) and publishes the grand total.
template <typename TOut>
__device__ __forceinline__ void scan_sums_body(TOut* __restrict__ sums, int num_tiles, TOut* __restrict__ total_out)
{
    __shared__ TOut warp_sums[SCAN_THREADS / 32];
    TOut carry = 0;
    for (int b0 = 0; b0 < num_tiles; b0 += SCAN_THREADS) {
        const int i = b0 + threadIdx.x;
        TOut v = (i < num_tiles) ? sums[i] : (TOut)0;
        TOut tot;
        TOut ex = block_excl_scan<TOut>(v, &tot, warp_sums);
        if (i < num_tiles) sums[i] = carry + ex;
        carry += tot;
    }
    if (threadIdx.x == 0 && total_out != nullptr) *total_out = carry;
}

template <typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_sums_kernel(TOut* __restrict__ sums, int num_tiles, TOut* __restrict__ total_out)
{
    scan_sums_body<TOut>(sums, num_tiles, total_out);
}

template <typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_sums_pair_kernel(TOut* __restrict__ sums, int num_tiles, TOut* __restrict__ total0, TOut* __restrict__ total1)
{
    scan_sums_body<TOut>(sums + (size_t)blockIdx.x * num_tiles, num_tiles, blockIdx.x ? total1 : total0);
}

template <typename TIn, typename TOut>
__device__ __forceinline__ void scan_apply_body(const TIn* in, const uint32_t* __restrict__ n_dev, int64_t n_host,
                                                const TOut* __restrict__ sums, TOut* out, TOut* out_copy = nullptr)
{
    __shared__ TOut warp_sums[SCAN_THREADS / 32];
    const int64_t n = scan_count(n_dev, n_host);
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    TOut v[SCAN_ITEMS];
    scan_load_items<TIn, TOut>(in, base, n, v);
    TOut s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++) s += v[i];
    TOut tot;
    TOut run = block_excl_scan<TOut>(s, &tot, warp_sums) + sums[blockIdx.x];
    scan_store_items<TOut>(out, base, n, run, v);
    if (out_copy != nullptr) scan_store_items<TOut>(out_copy, base, n, run, v);
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_kernel(const TIn* in, const uint32_t* __restrict__ n_dev, int64_t n_host,
                  const TOut* __restrict__ sums, TOut* out)
{
    scan_apply_body<TIn, TOut>(in, n_dev, n_host, sums, out);
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_pair_kernel(const TIn* in0, TOut* out0, const TIn* in1, TOut* out1, const uint32_t* __restrict__ n_dev, int64_t n_host,
                       const TOut* __restrict__ sums, TOut* copy0, TOut* copy1)
{
    scan_apply_body<TIn, TOut>(blockIdx.y ? in1 : in0, n_dev, n_host, sums + (size_t)blockIdx.y * gridDim.x, blockIdx.y ? out1 : out0,
                               blockIdx.y ? copy1 : copy0);
}

// sum of sums[0 .. blockIdx.x) by the whole block (and, from the last block, the grand total)
template <typename TOut>
__device__ __forceinline__ TOut scan_prefix_of_sums(const TOut* __restrict__ sums, int num_tiles, TOut* __restrict__ total_out)
{
    __shared__ TOut part[SCAN_THREADS / 32];
    __shared__ TOut result;
    const int mine = blockIdx.x;
    TOut s = 0;
    for (int i = threadIdx.x; i < mine; i += SCAN_THREADS) s += sums[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        TOut t = 0;
#pragma unroll
        for (int w = 0; w < SCAN_THREADS / 32; w++) t += part[w];
        result = t;
        if (total_out != nullptr && mine == num_tiles - 1) *total_out = t + sums[mine];
    }
    __syncthreads();
    return result;
}

template <typename TIn, typename TOut>
__device__ __forceinline__ void scan_apply_fused_body(const TIn* in, const uint32_t* __restrict__ n_dev, int64_t n_host,
                                                      const TOut* __restrict__ sums, int num_tiles, TOut* out, TOut* total_out,
                                                      TOut* out_copy = nullptr)
{
    __shared__ TOut warp_sums[SCAN_THREADS / 32];
    const int64_t n = scan_count(n_dev, n_host);
    // a tile past the (device-side) end has nothing to write; only the last block still adds up all sums for the total
    if ((int64_t)blockIdx.x * SCAN_TILE >= n && (int)blockIdx.x != num_tiles - 1) return;
    const TOut before = scan_prefix_of_sums<TOut>(sums, num_tiles, total_out);
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    TOut v[SCAN_ITEMS];
    scan_load_items<TIn, TOut>(in, base, n, v);
    TOut s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++) s += v[i];
    TOut tot;
    TOut run = block_excl_scan<TOut>(s, &tot, warp_sums) + before;
    scan_store_items<TOut>(out, base, n, run, v);
    if (out_copy != nullptr) scan_store_items<TOut>(out_copy, base, n, run, v);
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_fused_kernel(const TIn* in, const uint32_t* __restrict__ n_dev, int64_t n_host, const TOut* __restrict__ sums,
                        TOut* out, TOut* total_out)
{
    scan_apply_fused_body<TIn, TOut>(in, n_dev, n_host, sums, gridDim.x, out, total_out);
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_fused_pair_kernel(const TIn* in0, TOut* out0, TOut* total0, const TIn* in1, TOut* out1, TOut* total1,
                             const uint32_t* __restrict__ n_dev, int64_t n_host, const TOut* __restrict__ sums, TOut* copy0,
                             TOut* copy1)
{
    scan_apply_fused_body<TIn, TOut>(blockIdx.y ? in1 : in0, n_dev, n_host, sums + (size_t)blockIdx.y * gridDim.x, gridDim.x,
                                     blockIdx.y ? out1 : out0, blockIdx.y ? total1 : total0, blockIdx.y ? copy1 : copy0);
}

constexpr int SCAN_FUSED_MAX_TILES = 8192;  // above this the per-block summing of earlier tiles stops being negligible

static inline int scan_num_tiles(int64_t n_host) { return (int)((n_host + SCAN_TILE - 1) / SCAN_TILE); }

// `sums` must hold scan_num_tiles(n_host) elements of TOut.  `total_out` (device, may be null)
// receives the sum of all elements.
template <typename TIn, typename TOut>
static inline cudaError_t exclusive_scan(const TIn* in, TOut* out, const uint32_t* n_dev, int64_t n_host,
                                         TOut* sums, TOut* total_out, cudaStream_t stream)
{
    if (n_host <= 0) {
        if (total_out) return cudaMemsetAsync(total_out, 0, sizeof(TOut), stream);
        return cudaSuccess;
    }
    const int tiles = scan_num_tiles(n_host);
    scan_tile_sums_kernel<TIn, TOut><<<tiles, SCAN_THREADS, 0, stream>>>(in, n_dev, n_host, sums);
    if (tiles <= SCAN_FUSED_MAX_TILES) {
        scan_apply_fused_kernel<TIn, TOut><<<tiles, SCAN_THREADS, 0, stream>>>(in, n_dev, n_host, sums, out, total_out);
    } else {
        scan_sums_kernel<TOut><<<1, SCAN_THREADS, 0, stream>>>(sums, tiles, total_out);
        scan_apply_kernel<TIn, TOut><<<tiles, SCAN_THREADS, 0, stream>>>(in, n_dev, n_host, sums, out);
    }
    return cudaGetLastError();
}

// Two arrays of the same (possibly device-side) length in the same launches.  `sums` must hold
// 2 x scan_num_tiles(n_host) elements.  copy0 / copy1 (may be null): a second array that receives the same result.
template <typename TIn, typename TOut>
static inline cudaError_t exclusive_scan_pair(const TIn* in0, TOut* out0, TOut* total0, const TIn* in1, TOut* out1, TOut* total1,
                                              const uint32_t* n_dev, int64_t n_host, TOut* sums, cudaStream_t stream,
                                              TOut* copy0 = nullptr, TOut* copy1 = nullptr)
{
    if (n_host <= 0) return cudaSuccess;
    const int tiles = scan_num_tiles(n_host);
    scan_tile_sums_pair_kernel<TIn, TOut><<<dim3(tiles, 2), SCAN_THREADS, 0, stream>>>(in0, in1, n_dev, n_host, sums);
    if (tiles <= SCAN_FUSED_MAX_TILES) {
        scan_apply_fused_pair_kernel<TIn, TOut><<<dim3(tiles, 2), SCAN_THREADS, 0, stream>>>(in0, out0, total0, in1, out1, total1, n_dev,
                                                                                          n_host, sums, copy0, copy1);
    } else {
        scan_sums_pair_kernel<TOut><<<2, SCAN_THREADS, 0, stream>>>(sums, tiles, total0, total1);
        scan_apply_pair_kernel<TIn, TOut><<<dim3(tiles, 2), SCAN_THREADS, 0, stream>>>(in0, out0, in1, out1, n_dev, n_host, sums, copy0, copy1);
    }
    return cudaGetLastError();
}

}  // namespace dynb
