// Periodic cell-list radius graph for B200 (sm_100a).
//
// Replaces the reference's radius_graph_pbc_cuda_impl_ex
// (dynamis_state/src/csrc/graph/radius_graph_kernels.cu:479-934) behind the C ABI in dynb.h.
//
// Pipeline (one stream, no host synchronisation inside the plan):
//   rg_wrap        wrap positions into the unit cell, classify which periodic images each atom
//                  needs, per-block bounding box of all images           (ref :596-605, :18-67)
//   rg_target_bbox bounding box of the targets (only with a target subset)
//   rg_grid        one block: reduce the boxes, choose the cell grid on the device (ref :662-692)
//   rg_bin_count   histogram of images / targets per cell (atomics)      (ref :146-171)
//   scan           cell starts
//   rg_bin_scatter provisional slot inside each cell (atomic rank)
//   rg_bin_finalize deterministic order inside each cell, write packed source / target records
//   rg_pair<COUNT> per-target degree                                     (ref :197-258)
//   scan           edge offsets + total
//   rg_pair<FILL>  edges                                                 (ref :282-442)
//
// The edge SET is fixed by three predicates that are kept expression-for-expression identical to
// the reference (same operand order, compiled with the same default FMA contraction): the wrap,
// the periodic-image test with the image position, and d2 <= r2 && d2 > 1e-8f.  The cell grid
// only decides which pairs are examined and is free to differ.
//
// Work decomposition of rg_pair: one warp owns a group of group_cells x group_cells_y cells (x, y)
// and all targets inside.  It flattens the contiguous runs of neighbouring source records (one run
// per (y, z) row, one lane per run) into a dense shared-memory list once, then tests the targets two
// at a time against the list with one candidate per lane (conflict-free 16-byte shared loads, ballot +
// popc compaction).  Hits are parked in per-target lists and written out 32 edges at a time so that
// the 8-byte index stores of a warp cover one contiguous 256-byte run.  With a target subset the
// source images are first clipped to the targets' bounding box grown by the cutoff.

#include "common.cuh"
#include "scan.cuh"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace dynb {

// ------------------------------------------------------------------------------------------
// Device-resident plan header.  The first 64 bytes mirror dynb_rg_header.
// ------------------------------------------------------------------------------------------
struct DevHeader {
    unsigned long long E;
    unsigned long long M;
    uint32_t status;
    uint32_t max_degree;
    int32_t nx, ny, nz;
    int32_t group_cells;
    unsigned long long num_groups;
    long long reserved[2];
    // ---- internal -----------------------------------------------------------------------
    uint32_t ncell_plus1;
    int32_t pad;
    int32_t gx;
    int32_t group_cells_y;  // cells per warp work item along y (1 or 2)
    unsigned long long bb_min[3];  // ordered-integer images of the bounding box
    unsigned long long bb_max[3];
    double gmin[3];
    double res_inv;
    double clip_lo[3];  // source images outside [clip_lo, clip_hi] cannot reach any target and are dropped
    double clip_hi[3];
    uint32_t active_groups;  // entries of the list of groups that hold targets (target subsets only)
    uint32_t long_groups;    // entries of the list of groups whose candidate list is too long for the hit bits
};
static_assert(offsetof(DevHeader, ncell_plus1) == sizeof(dynb_rg_header), "public header prefix mismatch");

constexpr uint32_t RG_FATAL = DYNB_RG_SRC_OVERFLOW | DYNB_RG_BAD_TARGET | DYNB_RG_NONFINITE | DYNB_RG_SHIFT_RANGE;

template <typename T> struct Geom {
    T inv[9];
    T cell[9];
    T cf[3];
    int rep[3];
    int pbc[3];
};

// Rounded-once helpers (no contraction across them).
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float fma_rn(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ double fma_rn(double a, double b, double c) { return __fma_rn(a, b, c); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float floor_t(float a) { return floorf(a); }
__device__ __forceinline__ double floor_t(double a) { return floor(a); }
__device__ __forceinline__ bool finite_t(float a) { return isfinite(a); }
__device__ __forceinline__ bool finite_t(double a) { return isfinite(a); }

__device__ __forceinline__ unsigned long long ordered_any(float v) { return (unsigned long long)ordered_u32(v); }
__device__ __forceinline__ unsigned long long ordered_any(double v) { return ordered_u64(v); }
// the same keys in their natural width: 32 bits for float (one REDUX instruction reduces them over a warp)
__device__ __forceinline__ uint32_t ordered_key(float v) { return ordered_u32(v); }
__device__ __forceinline__ unsigned long long ordered_key(double v) { return ordered_u64(v); }
template <typename T> __device__ __forceinline__ double unordered_any(unsigned long long u);
template <> __device__ __forceinline__ double unordered_any<float>(unsigned long long u) { return (double)unordered_f32((uint32_t)u); }
template <> __device__ __forceinline__ double unordered_any<double>(unsigned long long u) { return unordered_f64(u); }

// K = 3 inner product exactly as an fp32/fp64 GEMM accumulates it: k-sequential FMA chain.
// The reference wraps positions with two at::mm calls (radius_graph_kernels.cu:602,605).
template <typename T> __device__ __forceinline__ T dot3_gemm(T a0, T b0, T a1, T b1, T a2, T b2)
{
    return fma_rn(a2, b2, fma_rn(a1, b1, mul_rn(a0, b0)));
}

// Image position, same expression shape as the reference's write_pbc_images_kernel (:122-128).
template <typename T>
__device__ __forceinline__ void image_pos(const Geom<T>& g, T px, T py, T pz, int dx, int dy, int dz, T& x, T& y, T& z)
{
    T shift_x = (T)dx * g.cell[0] + (T)dy * g.cell[3] + (T)dz * g.cell[6];
    T shift_y = (T)dx * g.cell[1] + (T)dy * g.cell[4] + (T)dz * g.cell[7];
    T shift_z = (T)dx * g.cell[2] + (T)dy * g.cell[5] + (T)dz * g.cell[8];
    x = px + shift_x;
    y = py + shift_y;
    z = pz + shift_z;
}

// image flags of an atom: bit d = "may be shifted up along d", bit 3+d = "may be shifted down along d"

template <typename T>
__device__ __forceinline__ uint32_t cell_of(const DevHeader& h, T x, T y, T z)
{
    const T ri = (T)h.res_inv;
    int cx = (int)floor_t((x - (T)h.gmin[0]) * ri);
    int cy = (int)floor_t((y - (T)h.gmin[1]) * ri);
    int cz = (int)floor_t((z - (T)h.gmin[2]) * ri);
    cx = max(0, min(cx, h.nx - 1));
    cy = max(0, min(cy, h.ny - 1));
    cz = max(0, min(cz, h.nz - 1));
    return (uint32_t)cx + (uint32_t)h.nx * ((uint32_t)cy + (uint32_t)h.ny * (uint32_t)cz);
}

constexpr int RG_MASK_SLOTS = 16;  // hit bits kept per lane and target (candidate lists up to 512 records)

// The cell grid of a plan and the shape of a warp's work item.  Chosen on the device from the bounding box of
// the data (rg_grid_kernel), or on the host from the cell when the box is periodic in all directions and every
// atom is a target (the images then fill a known box and the first two passes run as one).
struct GridChoice {
    int nx, ny, nz, pad, group_cells, group_cells_y, gx;
    uint32_t ncell_plus1;
    unsigned long long num_groups;
    double gmin[3];
    double res_inv;
};

// Cells of edge radius/1.99 scanned +-2 (as the reference, :662,776) unless that would need more than
// cell_capacity cells; then the cells grow, and once they are wider than the cutoff the scan shrinks to +-1.
__host__ __device__ inline void rg_choose_shape(GridChoice& gc, double avg, int cand_capacity, int force_sx, int force_sy, bool allow_wide);
// avg: expected sources per cell, for the shape of the work items.
__host__ __device__ inline void rg_choose_grid(const double lo[3], const double ext[3], double radius, long long cell_capacity,
                                               int cand_capacity, double M, double sources_per_volume, int force_sx, int force_sy,
                                               bool allow_wide, GridChoice& gc)
{
    double res = radius / 1.99;
    long long n[3];
    for (int it = 0; it < 400; it++) {
        double tot = 1.0;
        for (int k = 0; k < 3; k++) {
            double c = ceil(ext[k] / res);
            if (!(c >= 1.0)) c = 1.0;
            if (c > 2.0e9) c = 2.0e9;
            n[k] = (long long)c;
            tot *= c;
        }
        if (tot + 1.0 <= (double)cell_capacity) break;
        res *= 1.2;
        if (it == 399) { n[0] = n[1] = n[2] = 1; }
    }
    gc.nx = (int)n[0]; gc.ny = (int)n[1]; gc.nz = (int)n[2];
    const long long ncell = n[0] * n[1] * n[2];
    gc.ncell_plus1 = (uint32_t)(ncell + 1);
    const int pad = (res >= radius * 1.001) ? 1 : 2;
    gc.pad = pad;
    for (int k = 0; k < 3; k++) gc.gmin[k] = lo[k];
    gc.res_inv = 1.0 / res;
    rg_choose_shape(gc, sources_per_volume > 0.0 ? sources_per_volume * res * res * res : M / (double)ncell, cand_capacity, force_sx,
                    force_sy, allow_wide);
}

// cells per warp work item (Sx along x, Sy along y): as many target cells as possible while the
// expected dense candidate list stays within 1.5 shared-memory lists
// allow_wide: the mean is taken over a box that the sources fill.  With a target subset the grid can span far more
// cells than hold sources (a subdomain whose wrapped targets sit on both sides of the periodic box), the mean then
// says nothing about the lists, and the wide shapes — which sit just under the limit of the hit bits — stay out.
__host__ __device__ inline void rg_choose_shape(GridChoice& gc, double avg, int cand_capacity, int force_sx, int force_sy, bool allow_wide)
{
    const int pad = gc.pad;
    // measured on B200 (1 M-atom liquid, 1 M-atom fcc): 2 x 2 cells per warp beat 2 x 1 and 1 x 1 even when the
    // candidate list then needs a second chunk, and wider groups (3 or 4 cells along x, which lengthens every
    // candidate run instead of adding runs) beat 2 x 2 as long as the list keeps its hit bits: the work per group
    // (decode, run table, staging) is shared by more targets.  A list longer than the hit bits sends its group to
    // the slow writer, so the wide shapes are taken only with a margin (15 % on the mean density, four standard
    // deviations of a Poisson count) under that limit.
    const double budget = 1.5 * (double)cand_capacity;
    const int shapes[5][2] = {{4, 2}, {3, 2}, {2, 2}, {2, 1}, {1, 1}};
    int bestx = 1, besty = 1;
    for (int c = 0; c < 5; c++) {
        const int sx = shapes[c][0], sy = shapes[c][1];
        if ((sy + 2 * pad) * (2 * pad + 1) > 32) continue;  // one lane per candidate run
        if (sx > 2 && !allow_wide) continue;
        const double Lexp = (double)(sx + 2 * pad) * (double)(sy + 2 * pad) * (double)(2 * pad + 1) * (avg > 1e-6 ? avg : 1e-6);
        const bool fits = (sx > 2) ? (1.15 * Lexp + 4.0 * sqrt(Lexp) <= (double)(RG_MASK_SLOTS * 32)) : (Lexp <= budget);
        if (fits || c == 4) { bestx = sx; besty = sy; break; }
    }
    if (force_sx > 0) bestx = force_sx;
    if (force_sy > 0 && (force_sy + 2 * pad) * (2 * pad + 1) <= 32) besty = force_sy;
    if (bestx > gc.nx) bestx = gc.nx;
    if (besty > gc.ny) besty = gc.ny;
    gc.group_cells = bestx;
    gc.group_cells_y = besty;
    gc.gx = (gc.nx + bestx - 1) / bestx;
    const int gy = (gc.ny + besty - 1) / besty;
    gc.num_groups = (unsigned long long)gc.gx * (unsigned long long)gy * (unsigned long long)gc.nz;
}

__host__ __device__ inline void rg_store_grid(DevHeader& h, const GridChoice& gc)
{
    h.nx = gc.nx; h.ny = gc.ny; h.nz = gc.nz;
    h.ncell_plus1 = gc.ncell_plus1;
    h.pad = gc.pad;
    for (int k = 0; k < 3; k++) h.gmin[k] = gc.gmin[k];
    h.res_inv = gc.res_inv;
    h.group_cells = gc.group_cells;
    h.group_cells_y = gc.group_cells_y;
    h.gx = gc.gx;
    h.num_groups = gc.num_groups;
}

// cell_of for a grid that travels as a kernel argument: the same expression on the same numbers
template <typename T>
__device__ __forceinline__ uint32_t cell_of(const GridChoice& h, T x, T y, T z)
{
    const T ri = (T)h.res_inv;
    int cx = (int)floor_t((x - (T)h.gmin[0]) * ri);
    int cy = (int)floor_t((y - (T)h.gmin[1]) * ri);
    int cz = (int)floor_t((z - (T)h.gmin[2]) * ri);
    cx = max(0, min(cx, h.nx - 1));
    cy = max(0, min(cy, h.ny - 1));
    cz = max(0, min(cz, h.nz - 1));
    return (uint32_t)cx + (uint32_t)h.nx * ((uint32_t)cy + (uint32_t)h.ny * (uint32_t)cz);
}

// ------------------------------------------------------------------------------------------
// rg_wrap
// ------------------------------------------------------------------------------------------
// Squared distance with the rounding every pass must share (the contraction nvcc applies to
// dx*dx + dy*dy + dz*dz, written out so that no pass depends on the compiler's choice):
// fma(dz, dz, fma(dx, dx, dy * dy)).
template <typename T> __device__ __forceinline__ T dist2(T ax, T ay, T az, T sx, T sy, T sz)
{
    const T dx = sub_rn(ax, sx), dy = sub_rn(ay, sy), dz = sub_rn(az, sz);
    return fma_rn(dz, dz, fma_rn(dx, dx, mul_rn(dy, dy)));
}
// The same for two fp32 candidates at once with the packed fp32 instructions of sm_100 (each half is an
// IEEE round-to-nearest operation, so the halves equal dist2<float> bit for bit); one instruction issue
// per two tests.
__device__ __forceinline__ unsigned long long f32x2_pack(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void dist2_x2(unsigned long long ax2, unsigned long long ay2, unsigned long long az2,
                                         unsigned long long sx2, unsigned long long sy2, unsigned long long sz2,
                                         float& d_lo, float& d_hi)
{
    unsigned long long dx, dy, dz, d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(dx) : "l"(ax2), "l"(sx2));
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(dy) : "l"(ay2), "l"(sy2));
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(dz) : "l"(az2), "l"(sz2));
    asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(d) : "l"(dy));
    asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(d) : "l"(dx), "l"(d));
    asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(d) : "l"(dz), "l"(d));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d_lo), "=f"(d_hi) : "l"(d));
}

constexpr int WRAP_THREADS = 256;

// FUSED: the grid is known before the launch (gc, chosen on the host), so the images and the targets are counted
// into their cells here and no bounding box is gathered.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(WRAP_THREADS)
rg_wrap_kernel(const T* __restrict__ pos, int64_t N, Geom<T> g, int vec_ok, Vec4<T>* __restrict__ posw,
               int4* __restrict__ aff, DevHeader* __restrict__ h, unsigned long long* __restrict__ partials,
               const GridChoice gc, uint32_t* __restrict__ ccount, uint32_t* __restrict__ tccount)
{
    __shared__ T stage[WRAP_THREADS * 3];
    __shared__ unsigned long long red[6][WRAP_THREADS / 32];
    __shared__ unsigned int red_cnt[WRAP_THREADS / 32];

    const int64_t block_base = (int64_t)blockIdx.x * WRAP_THREADS;
    const int64_t i = block_base + threadIdx.x;
    const int64_t nblock = min((int64_t)WRAP_THREADS, N - block_base);

    // Coalesced 16-byte loads of this block's 3*nblock reals, then a conflict-free stride-3 read.
    {
        const T* src = pos + block_base * 3;
        const int nreal = (int)nblock * 3;
        constexpr int PER = 16 / (int)sizeof(T);
        if (vec_ok && nblock == WRAP_THREADS) {
            using V = typename std::conditional<sizeof(T) == 4, float4, double2>::type;
            const V* src4 = reinterpret_cast<const V*>(src);
            V* dst4 = reinterpret_cast<V*>(stage);
            for (int k = threadIdx.x; k < nreal / PER; k += WRAP_THREADS) dst4[k] = src4[k];
        } else {
            for (int k = threadIdx.x; k < nreal; k += WRAP_THREADS) stage[k] = src[k];
        }
    }
    __syncthreads();

    using Key = typename std::conditional<sizeof(T) == 4, uint32_t, unsigned long long>::type;
    Key mn[3] = {~(Key)0, ~(Key)0, ~(Key)0}, mx[3] = {0, 0, 0};
    unsigned int count = 0;
    uint32_t status = 0;

    if (i < N) {
        const T px = stage[threadIdx.x * 3 + 0], py = stage[threadIdx.x * 3 + 1], pz = stage[threadIdx.x * 3 + 2];
        T f[3], m[3];
#pragma unroll
        for (int k = 0; k < 3; k++) f[k] = floor_t(dot3_gemm(px, g.inv[k], py, g.inv[3 + k], pz, g.inv[6 + k]));
#pragma unroll
        for (int k = 0; k < 3; k++) m[k] = dot3_gemm(f[0], g.cell[k], f[1], g.cell[3 + k], f[2], g.cell[6 + k]);
        const T wx = sub_rn(px, m[0]), wy = sub_rn(py, m[1]), wz = sub_rn(pz, m[2]);

        if (!(finite_t(wx) && finite_t(wy) && finite_t(wz))) status |= DYNB_RG_NONFINITE;
        const T lim = (T)1048576.0;
        if (!(fabs(f[0]) < lim && fabs(f[1]) < lim && fabs(f[2]) < lim)) status |= DYNB_RG_SHIFT_RANGE;

        // Fractional coordinates of the wrapped position, reference expression (:36-38).
        T s[3];
        s[0] = wx * g.inv[0] + wy * g.inv[3] + wz * g.inv[6];
        s[1] = wx * g.inv[1] + wy * g.inv[4] + wz * g.inv[7];
        s[2] = wx * g.inv[2] + wy * g.inv[5] + wz * g.inv[8];
        uint32_t flags = 0;
#pragma unroll
        for (int d = 0; d < 3; d++) {
            if (g.pbc[d]) {
                if (!(s[d] >= g.cf[d])) flags |= (1u << d);                 // :55
                if (!(s[d] <= (T)1.0f - g.cf[d])) flags |= (8u << d);       // :58
            }
        }
        if (!(status & DYNB_RG_NONFINITE) && flags == 0) {
            // interior atom: only its own (0,0,0) image
            T x, y, z;
            image_pos(g, wx, wy, wz, 0, 0, 0, x, y, z);
            if (FUSED) atomicAdd(&ccount[cell_of(gc, x, y, z)], 1u);
            mn[0] = mx[0] = ordered_key(x);
            mn[1] = mx[1] = ordered_key(y);
            mn[2] = mx[2] = ordered_key(z);
            count = 1;
        } else if (!(status & DYNB_RG_NONFINITE)) {
            // the images an atom needs form a box of shifts (the flags are per axis and direction): walk
            // that box only, so that a warp runs as many rounds as its busiest atom has images, not (2 rep + 1)^3
            const int lo0 = (flags & 8u) ? -g.rep[0] : 0, hi0 = (flags & 1u) ? g.rep[0] : 0;
            const int lo1 = (flags & 16u) ? -g.rep[1] : 0, hi1 = (flags & 2u) ? g.rep[1] : 0;
            const int lo2 = (flags & 32u) ? -g.rep[2] : 0, hi2 = (flags & 4u) ? g.rep[2] : 0;
            for (int dx = lo0; dx <= hi0; dx++)
                for (int dy = lo1; dy <= hi1; dy++)
                    for (int dz = lo2; dz <= hi2; dz++) {
                        T x, y, z;
                        image_pos(g, wx, wy, wz, dx, dy, dz, x, y, z);
                        if (FUSED) atomicAdd(&ccount[cell_of(gc, x, y, z)], 1u);
                        const Key ox = ordered_key(x), oy = ordered_key(y), oz = ordered_key(z);
                        mn[0] = min(mn[0], ox); mx[0] = max(mx[0], ox);
                        mn[1] = min(mn[1], oy); mx[1] = max(mx[1], oy);
                        mn[2] = min(mn[2], oz); mx[2] = max(mx[2], oz);
                        count++;
                    }
        }
        Vec4<T> w;
        w.x = wx; w.y = wy; w.z = wz; w.w = bits_to_real((int32_t)flags, T());
        posw[i] = w;
        aff[i] = make_int4((int)f[0], (int)f[1], (int)f[2], (int)count);
        // every atom is a target, binned by its wrapped position (as rg_bin_kernel does)
        if (FUSED && !(status & DYNB_RG_NONFINITE)) atomicAdd(&tccount[cell_of(gc, wx, wy, wz)], 1u);
    }

    // block reduction
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int k = 0; k < 3; k++) {
            mn[k] = (Key)__reduce_min_sync(0xffffffffu, (unsigned)mn[k]);
            mx[k] = (Key)__reduce_max_sync(0xffffffffu, (unsigned)mx[k]);
        }
        count = __reduce_add_sync(0xffffffffu, count);
        status = __reduce_or_sync(0xffffffffu, status);
    } else {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                mn[k] = min(mn[k], (Key)__shfl_xor_sync(0xffffffffu, mn[k], o));
                mx[k] = max(mx[k], (Key)__shfl_xor_sync(0xffffffffu, mx[k], o));
            }
            count += __shfl_xor_sync(0xffffffffu, count, o);
            status |= __shfl_xor_sync(0xffffffffu, status, o);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 3; k++) {
            // "no image" stays the 64-bit identity of the minimum that rg_grid_kernel expects
            red[k][warp] = (mn[k] == ~(Key)0) ? ~0ull : (unsigned long long)mn[k];
            red[3 + k][warp] = (unsigned long long)mx[k];
        }
        red_cnt[warp] = count;
        if (status) atomicOr(&h->status, status);
    }
    __syncthreads();
    if (FUSED) {
        // the bounding box goes straight to the header (it only steers the shape of the work items, which is
        // settled three launches later): six fire-and-forget atomics per block
        if (threadIdx.x < 6) {
            unsigned long long v = red[threadIdx.x][0];
            for (int w = 1; w < WRAP_THREADS / 32; w++)
                v = (threadIdx.x < 3) ? min(v, red[threadIdx.x][w]) : max(v, red[threadIdx.x][w]);
            if (threadIdx.x < 3) atomicMin(&h->bb_min[threadIdx.x], v);
            else atomicMax(&h->bb_max[threadIdx.x - 3], v);
        }
        return;
    }
    // per-block partial results (bounding box, image count); rg_grid_kernel reduces them, so that no
    // block contends for a handful of header words
    if (threadIdx.x < 6) {
        unsigned long long v = red[threadIdx.x][0];
        for (int w = 1; w < WRAP_THREADS / 32; w++)
            v = (threadIdx.x < 3) ? min(v, red[threadIdx.x][w]) : max(v, red[threadIdx.x][w]);
        partials[(size_t)blockIdx.x * 8 + threadIdx.x] = v;
    } else if (threadIdx.x == 6) {
        unsigned long long c = 0;
        for (int w = 0; w < WRAP_THREADS / 32; w++) c += red_cnt[w];
        partials[(size_t)blockIdx.x * 8 + 6] = c;
    }
}

// Bounding box of the wrapped TARGET positions (only when a target subset is given): per-block
// partials, reduced by rg_grid_kernel.  Sources farther than the cutoff from that box are never
// needed, which keeps the grid and the image count small when a rank builds edges for its own
// atoms only.
template <typename T>
__global__ void __launch_bounds__(256)
rg_target_bbox_kernel(const int64_t* __restrict__ targets, int64_t Nt, int64_t N, const Vec4<T>* __restrict__ posw,
                      unsigned long long* __restrict__ partials)
{
    __shared__ unsigned long long red[6][8];
    unsigned long long v[6] = {~0ull, ~0ull, ~0ull, 0ull, 0ull, 0ull};
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < Nt) {
        const int64_t a = targets[i];
        if (a >= 0 && a < N) {
            const Vec4<T> w = posw[a];
            v[0] = v[3] = ordered_any(w.x);
            v[1] = v[4] = ordered_any(w.y);
            v[2] = v[5] = ordered_any(w.z);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < 3; k++) {
            v[k] = min(v[k], __shfl_xor_sync(0xffffffffu, v[k], o));
            v[3 + k] = max(v[3 + k], __shfl_xor_sync(0xffffffffu, v[3 + k], o));
        }
    if ((threadIdx.x & 31) == 0)
        for (int k = 0; k < 6; k++) red[k][threadIdx.x >> 5] = v[k];
    __syncthreads();
    if (threadIdx.x < 6) {
        unsigned long long a = red[threadIdx.x][0];
        for (int w = 1; w < 8; w++) a = (threadIdx.x < 3) ? min(a, red[threadIdx.x][w]) : max(a, red[threadIdx.x][w]);
        partials[(size_t)blockIdx.x * 8 + threadIdx.x] = a;
    }
}

// ------------------------------------------------------------------------------------------
// rg_grid: one thread chooses the grid.  Cells of edge radius/1.99 scanned +-2 (as the
// reference, :662,776) unless that would need more than cell_capacity cells; then the cells
// grow, and once they are wider than the cutoff the scan shrinks to +-1.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024)
rg_grid_kernel(DevHeader* h, double radius, long long src_capacity, long long cell_capacity, int cand_capacity,
               int force_sx, int force_sy, const unsigned long long* __restrict__ partials, int num_partials,
               const unsigned long long* __restrict__ tpartials, int num_tpartials)
{
    {   // reduce the per-block partials of rg_wrap_kernel into the header
        __shared__ unsigned long long red[7][32];
        unsigned long long v[7] = {~0ull, ~0ull, ~0ull, 0ull, 0ull, 0ull, 0ull};
#pragma unroll 4
        for (int b = threadIdx.x; b < num_partials; b += blockDim.x) {  // independent loads, several in flight
#pragma unroll
            for (int k = 0; k < 3; k++) {
                v[k] = min(v[k], partials[(size_t)b * 8 + k]);
                v[3 + k] = max(v[3 + k], partials[(size_t)b * 8 + 3 + k]);
            }
            v[6] += partials[(size_t)b * 8 + 6];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                v[k] = min(v[k], __shfl_xor_sync(0xffffffffu, v[k], o));
                v[3 + k] = max(v[3 + k], __shfl_xor_sync(0xffffffffu, v[3 + k], o));
            }
            v[6] += __shfl_xor_sync(0xffffffffu, v[6], o);
        }
        if ((threadIdx.x & 31) == 0)
            for (int k = 0; k < 7; k++) red[k][threadIdx.x >> 5] = v[k];
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int k = 0; k < 7; k++) {
                unsigned long long a = red[k][0];
                for (int w = 1; w < (int)(blockDim.x >> 5); w++)
                    a = (k < 3) ? min(a, red[k][w]) : (k < 6 ? max(a, red[k][w]) : a + red[k][w]);
                if (k < 3) h->bb_min[k] = a; else if (k < 6) h->bb_max[k - 3] = a; else h->M = a;
            }
        }
    }
    __shared__ unsigned long long tbox[6];
    {   // bounding box of the target subset (if any), same block reduction
        __shared__ unsigned long long tred[6][32];
        unsigned long long v[6] = {~0ull, ~0ull, ~0ull, 0ull, 0ull, 0ull};
#pragma unroll 4
        for (int b = threadIdx.x; b < num_tpartials; b += blockDim.x) {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                v[k] = min(v[k], tpartials[(size_t)b * 8 + k]);
                v[3 + k] = max(v[3 + k], tpartials[(size_t)b * 8 + 3 + k]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < 3; k++) {
                v[k] = min(v[k], __shfl_xor_sync(0xffffffffu, v[k], o));
                v[3 + k] = max(v[3 + k], __shfl_xor_sync(0xffffffffu, v[3 + k], o));
            }
        if ((threadIdx.x & 31) == 0)
            for (int k = 0; k < 6; k++) tred[k][threadIdx.x >> 5] = v[k];
        __syncthreads();
        if (threadIdx.x < 6) {
            unsigned long long a = tred[threadIdx.x][0];
            for (int w = 1; w < (int)(blockDim.x >> 5); w++)
                a = (threadIdx.x < 3) ? min(a, tred[threadIdx.x][w]) : max(a, tred[threadIdx.x][w]);
            tbox[threadIdx.x] = a;
        }
        __syncthreads();
    }
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (h->M > (unsigned long long)src_capacity) h->status |= DYNB_RG_SRC_OVERFLOW;
    for (int k = 0; k < 3; k++) { h->clip_lo[k] = -1.0e300; h->clip_hi[k] = 1.0e300; }
    if (h->M == 0 || (h->status & RG_FATAL)) {
        h->nx = h->ny = h->nz = 1;
        h->ncell_plus1 = 2;
        h->pad = 1;
        h->group_cells = 1;
        h->group_cells_y = 1;
        h->gx = 1;
        h->num_groups = 0;
        h->gmin[0] = h->gmin[1] = h->gmin[2] = 0.0;
        h->res_inv = 1.0;
        return;
    }
    double lo[3], ext[3];
    for (int k = 0; k < 3; k++) {
        lo[k] = unordered_any<T>(h->bb_min[k]) - 0.01;
        double hi = unordered_any<T>(h->bb_max[k]) + 0.01;
        if (num_tpartials > 0 && tbox[k] <= tbox[3 + k]) {
            // clip to the targets' box grown by the cutoff (with slack far above any rounding)
            const double margin = radius * 1.001 + 0.02;
            const double tlo = unordered_any<T>(tbox[k]) - margin, thi = unordered_any<T>(tbox[3 + k]) + margin;
            if (tlo > lo[k]) lo[k] = tlo;
            if (thi < hi) hi = thi;
            h->clip_lo[k] = lo[k];
            h->clip_hi[k] = hi;
            if (hi < lo[k]) hi = lo[k];
        }
        ext[k] = hi - lo[k];
    }
    GridChoice gc;
    rg_choose_grid(lo, ext, radius, cell_capacity, cand_capacity, (double)h->M, 0.0, force_sx, force_sy, num_tpartials == 0, gc);
    rg_store_grid(*h, gc);
}

// ------------------------------------------------------------------------------------------
// binning
// ------------------------------------------------------------------------------------------
template <typename T, bool SCATTER>
__global__ void __launch_bounds__(256, 5)
rg_bin_kernel(int64_t N, int64_t Nt, const int64_t* __restrict__ targets, Geom<T> g,
              const Vec4<T>* __restrict__ posw, DevHeader* __restrict__ hp,
              uint32_t* __restrict__ ccount, uint32_t* __restrict__ cfill,
              uint32_t* __restrict__ tccount, uint32_t* __restrict__ tcfill,
              uint4* __restrict__ srec, uint2* __restrict__ trec, long long src_capacity, int shape_cand_capacity)
{
    const DevHeader h = *hp;
    // the counting pass still runs when only the image capacity is short (it writes nothing but the cell counters): the
    // prefix sum's total then leaves the true number of images in header.M for the caller's second attempt
    if (h.status & (SCATTER ? RG_FATAL : (RG_FATAL & ~(uint32_t)DYNB_RG_SRC_OVERFLOW))) return;
    if (SCATTER && h.M > (unsigned long long)src_capacity) {
        // more images than the caller's buffers hold (header.M is the prefix sum's total by now; with a grid chosen on
        // the host this is the first place that knows): nothing is placed, the plan is repeated with a larger capacity
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(&hp->status, DYNB_RG_SRC_OVERFLOW);
        return;
    }
    if (SCATTER && shape_cand_capacity > 0 && blockIdx.x == 0 && threadIdx.x == 0) {
        // grid chosen on the host: the shape of the work items is settled here, from the number of images and the
        // bounding box they really fill (gathered while wrapping) — an atom cluster in a large periodic box is as
        // dense in its cells as it is, whatever the volume of the cell
        double vol_cells = 1.0;
        const double res = 1.0 / h.res_inv;
        const int nn[3] = {h.nx, h.ny, h.nz};
        for (int k = 0; k < 3; k++) {
            const double ext = unordered_any<T>(h.bb_max[k]) - unordered_any<T>(h.bb_min[k]) + 0.02;
            double cells = ceil(ext / res);
            if (!(cells >= 1.0)) cells = 1.0;
            if (cells > (double)nn[k]) cells = (double)nn[k];
            vol_cells *= cells;
        }
        GridChoice gc;
        gc.nx = h.nx; gc.ny = h.ny; gc.nz = h.nz; gc.pad = h.pad;
        rg_choose_shape(gc, (double)h.M / vol_cells, shape_cand_capacity, 0, 0, true);
        hp->group_cells = gc.group_cells;
        hp->group_cells_y = gc.group_cells_y;
        hp->gx = gc.gx;
        hp->num_groups = gc.num_groups;
    }
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) {
        const Vec4<T> w = posw[i];
        const uint32_t flags = (uint32_t)real_to_bits(w.w);
        const int k1 = 2 * g.rep[1] + 1, k2 = 2 * g.rep[2] + 1;
        // box of needed shifts (see rg_wrap_kernel); same (dx, dy, dz) order as a full walk
        const int lo0 = (flags & 8u) ? -g.rep[0] : 0, hi0 = (flags & 1u) ? g.rep[0] : 0;
        const int lo1 = (flags & 16u) ? -g.rep[1] : 0, hi1 = (flags & 2u) ? g.rep[1] : 0;
        const int lo2 = (flags & 32u) ? -g.rep[2] : 0, hi2 = (flags & 4u) ? g.rep[2] : 0;
        for (int dx = lo0; dx <= hi0; dx++)
            for (int dy = lo1; dy <= hi1; dy++)
                for (int dz = lo2; dz <= hi2; dz++) {
                    T x, y, z;
                    image_pos(g, w.x, w.y, w.z, dx, dy, dz, x, y, z);
                    if ((double)x < h.clip_lo[0] || (double)x > h.clip_hi[0] || (double)y < h.clip_lo[1] || (double)y > h.clip_hi[1] ||
                        (double)z < h.clip_lo[2] || (double)z > h.clip_hi[2])
                        continue;  // farther than the cutoff from every target
                    const uint32_t c = cell_of(h, x, y, z);
                    if (!SCATTER) {
                        atomicAdd(&ccount[c], 1u);
                    } else {
                        // the fill cursors start at the cells' first slots (the prefix sum wrote them there too):
                        // one atomic and one 16-byte record {key, cell} per image
                        const uint32_t slot = atomicAdd(&cfill[c], 1u);
                        const unsigned code = (unsigned)(((dx + g.rep[0]) * k1 + (dy + g.rep[1])) * k2 + (dz + g.rep[2]));
                        srec[slot] = make_uint4(code, (uint32_t)i, c, 0u);  // (atom, shift code) orders the images of a cell
                    }
                }
    }
    if (i < Nt) {
        const int64_t a = targets ? targets[i] : i;
        if (a < 0 || a >= N) {
            atomicOr(&hp->status, DYNB_RG_BAD_TARGET);
        } else {
            const Vec4<T> w = posw[a];
            const uint32_t c = cell_of(h, w.x, w.y, w.z);
            if (!SCATTER) {
                atomicAdd(&tccount[c], 1u);
            } else {
                const uint32_t slot = atomicAdd(&tcfill[c], 1u);
                trec[slot] = make_uint2((uint32_t)i, c);
            }
        }
    }
}

__device__ __forceinline__ uint32_t pack_shift_code(int ex, int ey, int ez)
{
    return (uint32_t)(ex + 512) | ((uint32_t)(ey + 512) << 10) | ((uint32_t)(ez + 512) << 20);
}

// Deterministic order inside each cell (ascending key) and the packed records.
template <typename T>
__global__ void __launch_bounds__(256)
rg_bin_finalize_kernel(int64_t N, int64_t Nt, const int64_t* __restrict__ targets, Geom<T> g,
                       const Vec4<T>* __restrict__ posw, const int4* __restrict__ aff,
                       DevHeader* __restrict__ hp, const uint32_t* __restrict__ cstart,
                       const uint32_t* __restrict__ tcstart, const uint4* __restrict__ srec, const uint2* __restrict__ trec,
                       Vec4<T>* __restrict__ spos, float* __restrict__ sxyz, long long sxyz_stride,
                       uint32_t* __restrict__ scode, uint2* __restrict__ smeta, Vec4<T>* __restrict__ tpos, int4* __restrict__ tmeta)
{
    if (hp->status & RG_FATAL) return;
    const unsigned long long M = hp->M;
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool has_s = j < (int64_t)M, has_t = j < Nt;
    // The loads are issued level by level for the source image and the target of this thread together: the two
    // records, then everything that depends only on a record (cell range, position and floor of the atom), then
    // the records of the cell for the rank; the kernel waits for memory, not for arithmetic.
    uint4 srj = make_uint4(0u, 0u, 0u, 0u);
    uint2 trj = make_uint2(0u, 0u);
    if (has_s) srj = srec[j];
    if (has_t) trj = trec[j];
    uint32_t sb = 0, se = 0, tb = 0, te = 0;
    Vec4<T> sw = {}, tw = {};
    int4 sff = make_int4(0, 0, 0, 0), tff = make_int4(0, 0, 0, 0);
    int64_t ta = 0;
    if (has_s) {
        sb = cstart[srj.z];
        se = cstart[srj.z + 1];
        sw = posw[srj.y];
        sff = aff[srj.y];
    }
    if (has_t) {
        tb = tcstart[trj.y];
        te = tcstart[trj.y + 1];
        ta = targets ? targets[trj.x] : (int64_t)trj.x;
        tw = posw[ta];
        tff = aff[ta];
    }
    if (has_s) {
        const unsigned long long key = ((unsigned long long)srj.y << 32) | srj.x;
        uint32_t rank = 0;
        for (uint32_t q = sb; q < se; q++) {
            const uint2 kq = *reinterpret_cast<const uint2*>(&srec[q]);
            rank += ((((unsigned long long)kq.y << 32) | kq.x) < key) ? 1u : 0u;
        }
        const int k1 = 2 * g.rep[1] + 1, k2 = 2 * g.rep[2] + 1;
        const uint32_t atom = srj.y;
        unsigned code = srj.x;
        const int dz = (int)(code % k2) - g.rep[2]; code /= k2;
        const int dy = (int)(code % k1) - g.rep[1]; code /= k1;
        const int dx = (int)code - g.rep[0];
        Vec4<T> r;
        image_pos(g, sw.x, sw.y, sw.z, dx, dy, dz, r.x, r.y, r.z);
        r.w = bits_to_real((int32_t)atom, T());
        const uint32_t at = sb + rank;
        spos[at] = r;
        if (sizeof(T) == 4 && sxyz != nullptr) {
            sxyz[at] = (float)r.x;
            sxyz[sxyz_stride + at] = (float)r.y;
            sxyz[2 * sxyz_stride + at] = (float)r.z;
        }
        const int ex = dx - sff.x, ey = dy - sff.y, ez = dz - sff.z;
        uint32_t packed = pack_shift_code(0, 0, 0);
        if (ex < -511 || ex > 511 || ey < -511 || ey > 511 || ez < -511 || ez > 511) atomicOr(&hp->status, DYNB_RG_SHIFT_RANGE);
        else packed = pack_shift_code(ex, ey, ez);
        scode[at] = packed;
        smeta[at] = make_uint2(atom, packed);
    }
    if (has_t) {
        const uint32_t ent = trj.x;
        uint32_t rank = 0;
        for (uint32_t q = tb; q < te; q++) rank += (trec[q].x < ent) ? 1u : 0u;
        Vec4<T> r;
        r.x = tw.x; r.y = tw.y; r.z = tw.z; r.w = bits_to_real((int32_t)ent, T());
        tpos[tb + rank] = r;
        tmeta[tb + rank] = make_int4((int)ta, tff.x, tff.y, tff.z);
    }
}

// ------------------------------------------------------------------------------------------
// rg_pair: the cell scan.
// ------------------------------------------------------------------------------------------
constexpr int PAIR_WARPS = 8;
constexpr int PAIR_THREADS = PAIR_WARPS * 32;
constexpr int PAIR_CAND_BYTES = 5120;  // dense candidate records per warp (320 float4 / 160 double4)
constexpr int PAIR_CODE_BYTES = 1280;  // packed shift code per candidate (up to 320)
constexpr int PAIR_LIST = 128;         // parked hits per target (uint16 each, two targets per warp)
// The pair kernels are launched with this many times the CTAs that fit the device at once: SMs do not
// all drain their share at the same speed, and a static one-wave split left the slowest SM 20-30 %
// behind the average; with several short waves the block scheduler evens that out.
constexpr int PAIR_GRID_WAVES = 8;
constexpr int RUN_FLAG_WORDS = 16;     // run-start bitmap of one staged chunk (up to 512 records)
constexpr int RUN_INDEX_BYTES = 32 * 4 + RUN_FLAG_WORDS * 4;
constexpr int PAIR_WARP_BYTES = PAIR_CAND_BYTES + PAIR_CODE_BYTES + PAIR_LIST * 4 + RUN_INDEX_BYTES;

// Flattened candidate list of a warp: lane r owns source run r (run_a = first record, run_off = place
// of the run in the flattened list).  To find the record behind flattened index jj, the non-empty
// runs are compacted into delta[] (record = delta[rank] + jj) and every chunk of the list gets a bitmap
// of the places where a run starts; the rank of the run that covers jj is then a population count.
__device__ __forceinline__ void runs_compact(int* delta, int run_a, int run_off, int run_len, uint32_t lt)
{
    const uint32_t nem = __ballot_sync(0xffffffffu, run_len > 0);
    if (run_len > 0) delta[__popc(nem & lt)] = run_a - run_off;
}
// Asynchronous global -> shared copies (LDGSTS): the records of a whole chunk are requested back to back
// without passing through registers; cp_async_wait_all() before the warp reads them.
template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* gsrc)
{
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(d), "l"(gsrc), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// returns the number of non-empty runs that start before cbeg; flags covers [cbeg, cbeg + 32 * RUN_FLAG_WORDS)
__device__ __forceinline__ int runs_flags(uint32_t* flags, int run_off, int run_len, int lane, int cbeg)
{
    if (lane < RUN_FLAG_WORDS) flags[lane] = 0u;
    __syncwarp();
    const int rel = run_off - cbeg;
    if (run_len > 0 && rel >= 0 && rel < 32 * RUN_FLAG_WORDS) atomicOr(&flags[rel >> 5], 1u << (rel & 31));
    const uint32_t before = __ballot_sync(0xffffffffu, run_len > 0 && rel < 0);
    __syncwarp();
    return __popc(before);
}

enum { MODE_COUNT = 0, MODE_FILL = 1, MODE_HALO = 2 };

// MODE_HALO: instead of counting or writing edges, record for every edge src -> dst whose
// endpoints have different owners that owner(dst) needs src (bit owner(dst) of needed[src]) and
// that dst has a foreign neighbour.  This is the edge loop of the reference's halo-map builder
// (dynamis_state/src/csrc/build_halo_maps.cpp:50-58, 127-138) without materialising the graph.
struct HaloArgs {
    const long long* owner;   // [n_atoms] rank of each atom
    uint32_t* needed;         // [n_atoms, words]
    unsigned char* has_foreign;  // [n_atoms]
    int words;
};

#ifndef DYNB_COUNT_UNROLL
#define DYNB_COUNT_UNROLL 1
#endif
constexpr int COUNT_UNROLL = DYNB_COUNT_UNROLL;  // unroll factor of the count pass's test loop (tuning knob at build time)

// Optional extras of the edge writers for the model-side glue: the shifts written with the caller's sign
// and the Cartesian shift of every edge, unit_shift @ cell, rounded like a K = 3 float GEMM
// (products and sums of torch.matmul(unit_shifts, cell): fma(u2, c2, fma(u1, c1, u0 * c0))).
struct GlueArgs {
    float* cart;              // [E,3] or nullptr
    const long long* id_map;  // [n_atoms] ids to write instead of the atom indices (local -> global), or nullptr
    int negate;               // 1: write -shift
    float c[9];               // cell, row-major
};
__device__ __forceinline__ void glue_write(const GlueArgs& g, float* __restrict__ shifts, long long e, int ix, int iy, int iz)
{
    if (g.negate) { ix = -ix; iy = -iy; iz = -iz; }
    const float u0 = (float)ix, u1 = (float)iy, u2 = (float)iz;
    shifts[3 * e + 0] = u0;
    shifts[3 * e + 1] = u1;
    shifts[3 * e + 2] = u2;
    if (g.cart != nullptr) {
#pragma unroll
        for (int k = 0; k < 3; k++)
            g.cart[3 * e + k] = __fmaf_rn(u2, g.c[6 + k], __fmaf_rn(u1, g.c[3 + k], __fmul_rn(u0, g.c[k])));
    }
}

template <typename T> struct PairParams {
    DevHeader* h;
    const uint32_t* cstart;
    const uint32_t* tcstart;
    const Vec4<T>* spos;
    const float* sxyz;        // fp32 only: coordinates of the source records as three arrays, each sxyz_stride long
    long long sxyz_stride;
    const uint32_t* scode;    // packed (shift - floor(frac) of the source atom), 10 bits per axis, bias 512
    const Vec4<T>* tpos;
    const int4* tmeta;
    uint32_t* tcount;         // [Nt+1] degree per sorted target; running cursor in FILL
    const long long* toffset; // [Nt+1]
    unsigned short* hitmask;  // [Nt, 32] per lane: bit s set if candidate 32 s + lane is a neighbour (written by COUNT)
    const uint2* smeta;       // [M] {atom id, packed shift code} per source record
    int32_t* counts_out;      // [Nt] degrees in caller order, or nullptr
    const uint32_t* glist;    // groups that hold at least one target (h->active_groups entries), or nullptr = all groups
    uint32_t* long_list;      // groups whose candidate list exceeds the hit bits (h->long_groups entries, written by COUNT)
    T r2;
};
// The plan stores its PairParams inside the workspace (after the header) so that the fill call
// needs nothing but the workspace pointer.
constexpr int64_t RG_PARAMS_OFFSET = 512;
constexpr int64_t RG_HEADER_BYTES = 1024;

// With a target subset (a rank building edges for the atoms it owns) the grid may span far more cells than
// hold targets — a subdomain that touches the periodic boundary has wrapped targets on both sides of the box
// and its grid covers the whole box.  The cell-scan kernels then walk a list of the groups that hold targets
// instead of all groups.  The order of the list is not defined (it only distributes the work; every target's
// output place is fixed by the offsets).
template <typename T>
__global__ void __launch_bounds__(256)
rg_group_list_kernel(const PairParams<T>* __restrict__ params_dev, uint32_t* __restrict__ glist)
{
    const PairParams<T> p = *params_dev;
    DevHeader* hp = p.h;
    if (hp->status & RG_FATAL) return;
    const int nx = hp->nx, ny = hp->ny, S = hp->group_cells, Sy = hp->group_cells_y;
    const uint32_t gx = (uint32_t)hp->gx;
    const uint32_t gy = (uint32_t)((ny + Sy - 1) / Sy);
    const uint32_t num_groups = (uint32_t)hp->num_groups;
    const int lane = threadIdx.x & 31;
    for (uint32_t g0 = (blockIdx.x * blockDim.x + threadIdx.x) & ~31u; g0 < num_groups; g0 += gridDim.x * blockDim.x) {
        const uint32_t grp = g0 + lane;
        bool has = false;
        if (grp < num_groups) {
            const uint32_t row = grp / gx;
            const int ix = (int)(grp - row * gx);
            const int cz = (int)(row / gy), iy = (int)(row - (uint32_t)cz * gy);
            const int cx0 = ix * S, cx1 = min(cx0 + S, nx) - 1;
            const int cy0 = iy * Sy, cy1 = min(cy0 + Sy, ny) - 1;
            has = p.tcstart[((uint32_t)cz * ny + cy0) * nx + cx0] != p.tcstart[((uint32_t)cz * ny + cy0) * nx + cx1 + 1];
            if (!has && cy1 > cy0)
                has = p.tcstart[((uint32_t)cz * ny + cy1) * nx + cx0] != p.tcstart[((uint32_t)cz * ny + cy1) * nx + cx1 + 1];
        }
        const uint32_t m = __ballot_sync(0xffffffffu, has);
        uint32_t base = 0;
        if (lane == 0 && m) base = atomicAdd(&hp->active_groups, (uint32_t)__popc(m));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (has) glist[base + __popc(m & lanemask_lt())] = grp;
    }
}

template <typename T, int MODE, bool BYVAL>
__global__ void __launch_bounds__(PAIR_THREADS, 4)
rg_pair_kernel(const PairParams<T>* __restrict__ params_dev, const PairParams<T> params_val, long long* __restrict__ ei,
               float* __restrict__ shifts, T* __restrict__ d2out, const long long E, const HaloArgs halo, const int skip_if_masks,
               const GlueArgs glue)
{
    // BYVAL: the launch has the record at hand and passes it as a kernel argument; its fields are then operands
    // of the instructions instead of registers loaded (and, under register pressure, reloaded) from the workspace
    PairParams<T> params_loaded;
    if constexpr (!BYVAL) params_loaded = *params_dev;
    const PairParams<T>& p = BYVAL ? params_val : params_loaded;
    extern __shared__ __align__(32) unsigned char smem_raw[];
    constexpr int CAP = PAIR_CAND_BYTES / (int)sizeof(Vec4<T>);
    // The fp32 count pass keeps its candidates as three arrays of coordinates (no atom ids, no shift codes: the
    // space of both holds a whole list with hit bits) laid out for the packed distance test: the 8 bytes that
    // lane l reads for block b hold the coordinate of candidates 64 b + l and 64 b + 32 + l.
    constexpr bool PACKED = (MODE == MODE_COUNT) && sizeof(T) == 4;
    constexpr int PK = RG_MASK_SLOTS * 32;
    constexpr int CAPX = PACKED ? PK : CAP;
    static_assert(3 * 4 * PK <= PAIR_CAND_BYTES + PAIR_CODE_BYTES, "packed candidates must fit the record and code space");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* wbase = smem_raw + warp * PAIR_WARP_BYTES;
    Vec4<T>* cand = reinterpret_cast<Vec4<T>*>(wbase);
    float* xs = reinterpret_cast<float*>(wbase);
    uint32_t* codes = reinterpret_cast<uint32_t*>(wbase + PAIR_CAND_BYTES);
    unsigned short* listA = reinterpret_cast<unsigned short*>(wbase + PAIR_CAND_BYTES + PAIR_CODE_BYTES);
    unsigned short* listB = listA + PAIR_LIST;
    int* delta = reinterpret_cast<int*>(wbase + PAIR_CAND_BYTES + PAIR_CODE_BYTES + PAIR_LIST * 4);
    uint32_t* flags = reinterpret_cast<uint32_t*>(delta + 32);
    const uint32_t le = lanemask_lt() | (1u << (threadIdx.x & 31));

    DevHeader* hp = p.h;
    if (hp->status & RG_FATAL) return;
    // behind rg_fillmask_kernel this pass writes only the groups whose candidate list was too long for the hit bits
    const bool long_only = (MODE == MODE_FILL) && skip_if_masks;
    if (long_only && hp->long_groups == 0u) return;
    int warp_max_slots = 0, warp_max_degree = 0;
    const int nx = hp->nx, ny = hp->ny, nz = hp->nz, S = hp->group_cells, Sy = hp->group_cells_y, pad = hp->pad;
    const uint32_t gx = (uint32_t)hp->gx;
    const uint32_t gy = (uint32_t)((ny + Sy - 1) / Sy);
    const uint32_t num_groups = long_only ? hp->long_groups
                                          : (p.glist ? hp->active_groups : (uint32_t)hp->num_groups);  // < 2^31: never more groups than cells
    const int Wd = 2 * pad + 1, Wy = Sy + 2 * pad, nrun = Wy * Wd;
    const int lane_dy = (lane % Wy) - pad, lane_dz = (lane / Wy) - pad;
    const T r2 = p.r2;
    const T eps = (T)1e-8f;
    const uint32_t lt = lanemask_lt();

    const uint32_t nwarps = gridDim.x * PAIR_WARPS;
    for (uint32_t gi = blockIdx.x * PAIR_WARPS + warp; gi < num_groups; gi += nwarps) {
        const uint32_t grp = long_only ? p.long_list[gi] : (p.glist ? p.glist[gi] : gi);
        const uint32_t row = grp / gx;
        const int ix = (int)(grp - row * gx);
        const int cz = (int)(row / gy), iy = (int)(row - (uint32_t)cz * gy);
        const int cx0 = ix * S, cx1 = min(cx0 + S, nx) - 1;
        const int cy0 = iy * Sy, cy1 = min(cy0 + Sy, ny) - 1;
        // targets: one contiguous run per target row
        uint32_t tb[2], te[2];
        tb[0] = p.tcstart[((uint32_t)cz * ny + cy0) * nx + cx0];
        te[0] = p.tcstart[((uint32_t)cz * ny + cy0) * nx + cx1 + 1];
        tb[1] = te[1] = 0;
        if (cy1 > cy0) {
            tb[1] = p.tcstart[((uint32_t)cz * ny + cy1) * nx + cx0];
            te[1] = p.tcstart[((uint32_t)cz * ny + cy1) * nx + cx1 + 1];
        }
        if (tb[0] == te[0] && tb[1] == te[1]) continue;

        // contiguous source runs: lane r owns run (y row, z row)
        int run_a = 0, run_len = 0;
        if (lane < nrun) {
            const int yy = cy0 + lane_dy, zz = cz + lane_dz;
            if (yy >= 0 && yy < ny && yy <= cy1 + pad && zz >= 0 && zz < nz) {
                const uint32_t b = ((uint32_t)zz * ny + yy) * nx;
                const uint32_t a = p.cstart[b + max(cx0 - pad, 0)];
                const uint32_t e = p.cstart[b + min(cx1 + pad, nx - 1) + 1];
                run_a = (int)a;
                run_len = (int)(e - a);
            }
        }
        int L;
        const int run_off = warp_excl_scan(run_len, lane, &L);
        const int nslots_total = (L + 31) >> 5;
        __syncwarp();
        runs_compact(delta, run_a, run_off, run_len, lt);
        const bool write_masks = (MODE == MODE_COUNT) && nslots_total <= RG_MASK_SLOTS;
        warp_max_slots = max(warp_max_slots, nslots_total);
        if (MODE == MODE_COUNT && nslots_total > RG_MASK_SLOTS && lane == 0) p.long_list[atomicAdd(&hp->long_groups, 1u)] = grp;

        for (int cbeg = 0, chunk = 0; cbeg < L; cbeg += CAPX, chunk++) {
            const int clen = min(CAPX, L - cbeg);
            const int clen32 = (clen + 31) & ~31;
            const bool more_chunks = cbeg + CAPX < L;
            // dense staging: slot j of the list holds flattened candidate cbeg + j; all loads of a chunk are
            // independent
            int rank_base = runs_flags(flags, run_off, run_len, lane, cbeg);
            if constexpr (PACKED) {
                // Per 64 candidates two rounds; in each the lower half-warp takes 16 candidates of the block's
                // first 32 and the upper half-warp 16 of its second 32, so that the 32 four-byte stores of a
                // round fall into 32 different banks and each half-warp reads 64 contiguous bytes per array.
                const int half = lane >> 4, l16 = lane & 15;
                for (int blk = 0; blk * 64 < clen; blk++) {
                    const uint32_t w0 = flags[2 * blk], w1 = flags[2 * blk + 1];
                    const uint32_t word = half ? w1 : w0;
                    const int base = rank_base + (half ? __popc(w0) : 0);
                    rank_base += __popc(w0) + __popc(w1);
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const int bitpos = i * 16 + l16;
                        const int j = blk * 64 + half * 32 + bitpos;
                        if (j < clen) {
                            const int r = base + __popc(word & ((2u << bitpos) - 1u)) - 1;
                            const float* src = p.sxyz + (delta[r] + cbeg + j);
                            float* dst = &xs[blk * 64 + bitpos * 2 + half];
                            cp_async<4>(dst, src);
                            cp_async<4>(dst + PK, src + p.sxyz_stride);
                            cp_async<4>(dst + 2 * PK, src + 2 * p.sxyz_stride);
                        }
                    }
                }
            } else {
            for (int j = lane, sw = 0; j < clen32; j += 32, sw++) {
                const uint32_t word = flags[sw];
                const int r = rank_base + __popc(word & le) - 1;
                rank_base += __popc(word);
                if (j < clen) {
                    const int gidx = delta[r] + cbeg + j;
                    if (sizeof(Vec4<T>) == 16) {
                        cp_async<16>(&cand[j], &p.spos[gidx]);  // w = atom id
                    } else {
                        cp_async<16>(&cand[j], &p.spos[gidx]);
                        cp_async<16>(reinterpret_cast<char*>(&cand[j]) + 16, reinterpret_cast<const char*>(&p.spos[gidx]) + 16);
                    }
                    if (MODE == MODE_FILL) cp_async<4>(&codes[j], &p.scode[gidx]);
                }
            }
            }
            if constexpr (PACKED) {
                // x alone keeps a padding slot out of every cutoff (its distance is infinite or not a number)
                for (int j = clen + lane; j < ((clen + 63) & ~63); j += 32) xs[(j >> 6) * 64 + (j & 31) * 2 + ((j >> 5) & 1)] = 3.0e38f;
            } else if (clen + lane < clen32) {
                Vec4<T> c;
                c.x = c.y = c.z = (T)3.0e38f;  // never within the cutoff
                c.w = (T)0;
                cand[clen + lane] = c;
            }
            cp_async_wait_all();
            __syncwarp();

          if constexpr (MODE == MODE_COUNT) {
            // the targets of both rows of the group as one list, two targets per candidate load
            const uint32_t n0 = te[0] - tb[0], ntot = n0 + (te[1] - tb[1]);
            for (uint32_t k = 0; k < ntot; k += 2) {
                const bool has2 = (k + 1 < ntot);
                const uint32_t kb = has2 ? k + 1 : k;
                const uint32_t tA = (k < n0) ? tb[0] + k : tb[1] + (k - n0);
                const uint32_t tB = (kb < n0) ? tb[0] + kb : tb[1] + (kb - n0);
                const Vec4<T> tpA = p.tpos[tA];
                const Vec4<T> tpB = p.tpos[tB];
                const T ax = tpA.x, ay = tpA.y, az = tpA.z, bx = tpB.x, by = tpB.y, bz = tpB.z;
                // lane l keeps, for each of its candidates l, 32 + l, 64 + l, ..., one hit bit per target; the
                // bits are stored so that the edge-writing pass need not repeat the distance tests.  A list too
                // long for the bits is only counted.
                unsigned short* mrowA = p.hitmask + (size_t)tA * 32;
                unsigned short* mrowB = p.hitmask + (size_t)tB * 32;
                uint32_t bitsA = 0, bitsB = 0;
                int ca = 0, cb = 0;
                if (chunk != 0) {
                    if (write_masks) {
                        bitsA = mrowA[lane];
                        bitsB = mrowB[lane];
                    } else {
                        ca = (int)p.tcount[tA];
                        cb = has2 ? (int)p.tcount[tB] : 0;
                    }
                }
                uint32_t bit = 1u << (cbeg >> 5);
                if constexpr (PACKED) {
                    const unsigned long long ax2 = f32x2_pack(ax, ax), ay2 = f32x2_pack(ay, ay), az2 = f32x2_pack(az, az);
                    const unsigned long long bx2 = f32x2_pack(bx, bx), by2 = f32x2_pack(by, by), bz2 = f32x2_pack(bz, bz);
                    const unsigned long long* x2 = reinterpret_cast<const unsigned long long*>(xs) + lane;
                    const int nblk = (clen + 63) >> 6;
                    int na = 0, nb = 0;
#pragma unroll COUNT_UNROLL
                    for (int blk = 0; blk < nblk; blk++) {
                        const unsigned long long sx2 = x2[blk * 32], sy2 = x2[PK / 2 + blk * 32], sz2 = x2[PK + blk * 32];
                        float a0, a1, b0, b1;
                        dist2_x2(ax2, ay2, az2, sx2, sy2, sz2, a0, a1);
                        dist2_x2(bx2, by2, bz2, sx2, sy2, sz2, b0, b1);
                        const bool ha0 = (a0 <= r2) && (a0 > eps), ha1 = (a1 <= r2) && (a1 > eps);
                        const bool hb0 = (b0 <= r2) && (b0 > eps), hb1 = (b1 <= r2) && (b1 > eps);
                        if (write_masks) {
                            bitsA |= (ha0 ? bit : 0u) | (ha1 ? (bit << 1) : 0u);
                            bitsB |= (hb0 ? bit : 0u) | (hb1 ? (bit << 1) : 0u);
                            bit <<= 2;
                        } else {
                            na += (ha0 ? 1 : 0) + (ha1 ? 1 : 0);
                            nb += (hb0 ? 1 : 0) + (hb1 ? 1 : 0);
                        }
                    }
                    if (!write_masks) {
                        ca += __reduce_add_sync(0xffffffffu, na);
                        cb += __reduce_add_sync(0xffffffffu, nb);
                    }
                } else {
                    int na = 0, nb = 0;
#pragma unroll COUNT_UNROLL
                    for (int kk = 0; kk < clen32; kk += 32) {
                        const Vec4<T> c = cand[kk + lane];
                        const T dA = dist2<T>(ax, ay, az, c.x, c.y, c.z);
                        const T dB = dist2<T>(bx, by, bz, c.x, c.y, c.z);
                        const bool hA = (dA <= r2) && (dA > eps), hB = (dB <= r2) && (dB > eps);
                        if (write_masks) {
                            bitsA |= hA ? bit : 0u;
                            bitsB |= hB ? bit : 0u;
                            bit <<= 1;
                        } else {
                            na += hA ? 1 : 0;
                            nb += hB ? 1 : 0;
                        }
                    }
                    if (!write_masks) {
                        ca += __reduce_add_sync(0xffffffffu, na);
                        cb += __reduce_add_sync(0xffffffffu, nb);
                    }
                }
                if (write_masks) {
                    mrowA[lane] = (unsigned short)bitsA;
                    if (has2) mrowB[lane] = (unsigned short)bitsB;
                    ca = __reduce_add_sync(0xffffffffu, __popc(bitsA));
                    cb = __reduce_add_sync(0xffffffffu, __popc(bitsB));
                }
                if (lane == 0) {
                    p.tcount[tA] = (uint32_t)ca;
                    if (has2) p.tcount[tB] = (uint32_t)cb;
                    if (!more_chunks && p.counts_out != nullptr) {  // degree in caller order (tpos.w = entry)
                        p.counts_out[real_to_bits(tpA.w)] = ca;
                        if (has2) p.counts_out[real_to_bits(tpB.w)] = cb;
                    }
                }
                if (!more_chunks) warp_max_degree = max(warp_max_degree, max(ca, has2 ? cb : 0));
            }
          } else {
#pragma unroll
          for (int yr = 0; yr < 2; yr++) {
            const uint32_t t0 = tb[yr], t1 = te[yr];
            // two targets share every candidate load
            for (uint32_t t = t0; t < t1; t += 2) {
                const bool has2 = (t + 1 < t1);
                const Vec4<T> tpA = p.tpos[t];
                const Vec4<T> tpB = p.tpos[has2 ? t + 1 : t];
                const T ax = tpA.x, ay = tpA.y, az = tpA.z, bx = tpB.x, by = tpB.y, bz = tpB.z;
                int prodA = 0, prodB = 0;
                if (chunk != 0 && MODE != MODE_HALO) {
                    prodA = (int)p.tcount[t];
                    prodB = has2 ? (int)p.tcount[t + 1] : 0;
                }
                {
                    int4 tmA = p.tmeta[t];
                    int4 tmB = p.tmeta[has2 ? t + 1 : t];
                    long long baseA = 0, baseB = 0, ownA = 0, ownB = 0;
                    bool foreignA = false, foreignB = false;
                    if (MODE == MODE_FILL) {
                        baseA = p.toffset[t];
                        baseB = p.toffset[has2 ? t + 1 : t];
                    } else {
                        ownA = halo.owner[tmA.x];
                        ownB = halo.owner[tmB.x];
                    }
                    int n = 0, nB = 0;  // parked hits of target A / target B
                    for (int k = 0; k < clen32; k += 32) {
                        const int j = k + lane;
                        const Vec4<T> c = cand[j];
                        const T dA = dist2<T>(ax, ay, az, c.x, c.y, c.z);
                        const T dB = dist2<T>(bx, by, bz, c.x, c.y, c.z);
                        const bool hitA = (dA <= r2) && (dA > eps);
                        const bool hitB = has2 && (dB <= r2) && (dB > eps);
                        if (MODE == MODE_HALO) {
                            if (hitA || hitB) {
                                const int a = real_to_bits(c.w);
                                const long long oa = halo.owner[a];
                                if (hitA && oa != ownA) {
                                    uint32_t* wd = &halo.needed[(long long)a * halo.words + (ownA >> 5)];
                                    const uint32_t bit = 1u << (ownA & 31);
                                    if (!(*wd & bit)) atomicOr(wd, bit);
                                    foreignA = true;
                                }
                                if (hitB && oa != ownB) {
                                    uint32_t* wd = &halo.needed[(long long)a * halo.words + (ownB >> 5)];
                                    const uint32_t bit = 1u << (ownB & 31);
                                    if (!(*wd & bit)) atomicOr(wd, bit);
                                    foreignB = true;
                                }
                            }
                        } else {
                            // each target parks the slots of its hits in its own half of the list; the index in
                            // the half is the position inside the target's edge run since the last write-out
                            const uint32_t mA = __ballot_sync(0xffffffffu, hitA);
                            const uint32_t mB = __ballot_sync(0xffffffffu, hitB);
                            if (hitA) listA[n + __popc(mA & lt)] = (unsigned short)j;
                            if (hitB) listB[nB + __popc(mB & lt)] = (unsigned short)j;
                            n += __popc(mA);
                            nB += __popc(mB);
                            if (n > PAIR_LIST - 32 || nB > PAIR_LIST - 32 || k + 32 >= clen32) {
                                __syncwarp();
#pragma unroll
                                for (int sel = 0; sel < 2; sel++) {
                                    const int cntX = sel ? nB : n;
                                    const unsigned short* lx = sel ? listB : listA;
                                    const int4 tm = sel ? tmB : tmA;
                                    const long long bX = (sel ? baseB + prodB : baseA + prodA);
                                    for (int i = lane; i < cntX; i += 32) {
                                        const int jh = lx[i];
                                        const Vec4<T> ch = cand[jh];
                                        const uint32_t code = codes[jh];
                                        const long long e = bX + i;
                                        const long long sa = (long long)real_to_bits(ch.w);
                                        ei[e] = glue.id_map ? glue.id_map[sa] : sa;
                                        ei[E + e] = glue.id_map ? glue.id_map[tm.x] : (long long)tm.x;
                                        glue_write(glue, shifts, e, (int)(code & 1023u) - 512 + tm.y, (int)((code >> 10) & 1023u) - 512 + tm.z,
                                                   (int)((code >> 20) & 1023u) - 512 + tm.w);
                                        if (d2out != nullptr) {
                                            const T tx = sel ? bx : ax, ty = sel ? by : ay, tz = sel ? bz : az;
                                            d2out[e] = dist2<T>(tx, ty, tz, ch.x, ch.y, ch.z);
                                        }
                                    }
                                }
                                prodA += n;
                                prodB += nB;
                                n = 0;
                                nB = 0;
                                __syncwarp();
                            }
                        }
                    }
                    if (MODE == MODE_FILL) {
                        if (more_chunks && lane == 0) {
                            p.tcount[t] = (uint32_t)prodA;
                            if (has2) p.tcount[t + 1] = (uint32_t)prodB;
                        }
                    } else {
                        if (__any_sync(0xffffffffu, foreignA) && lane == 0) halo.has_foreign[tmA.x] = 1;
                        if (has2 && __any_sync(0xffffffffu, foreignB) && lane == 0) halo.has_foreign[tmB.x] = 1;
                    }
                }
            }
          }
        }
          }
        // a group whose neighbourhood holds no source at all still owes its targets a zero
        if (MODE == MODE_COUNT && L == 0) {
            for (int yr = 0; yr < 2; yr++)
                for (uint32_t t = tb[yr] + lane; t < te[yr]; t += 32) p.tcount[t] = 0;
        }
    }
    if (MODE == MODE_COUNT) {  // largest degree: one atomic per CTA
        __shared__ int s_max_degree;
        if (threadIdx.x == 0) s_max_degree = 0;
        __syncthreads();
        if (lane == 0 && warp_max_degree > 0) atomicMax(&s_max_degree, warp_max_degree);
        __syncthreads();
        if (threadIdx.x == 0 && s_max_degree > 0) atomicMax(&hp->max_degree, (uint32_t)s_max_degree);
    }
    // a candidate list too long for the hit bits: the edge writer has to recompute distances
    if (MODE == MODE_COUNT && lane == 0 && warp_max_slots > RG_MASK_SLOTS) atomicMax(&hp->reserved[0], (long long)warp_max_slots);
}

// ------------------------------------------------------------------------------------------
// Edge writer driven by the hit masks of the counting pass.  When no group's candidate list is longer
// than RG_MASK_SLOTS * 32 records (the usual case: about 27 cells of 8-16 atoms) and the caller does
// not ask for distances, the edges follow from the masks alone: a warp stages {atom id, shift code}
// of its group's candidates, reads each target's mask words and writes the edge run.  No position is
// loaded and no distance is recomputed, and the edge order is the one rg_pair_kernel<FILL> gives.
// ------------------------------------------------------------------------------------------
constexpr int FM_META = RG_MASK_SLOTS * 32;                       // staged candidate records per warp
constexpr int FM_WARP_BYTES = FM_META * 8 + FM_META * 2 + RUN_INDEX_BYTES;    // records + one parked slot per possible hit

template <typename T, bool GLUE>
__global__ void __launch_bounds__(PAIR_THREADS, 4)
rg_fillmask_kernel(const PairParams<T>* __restrict__ params_dev, long long* __restrict__ ei, float* __restrict__ shifts,
                   const long long E, const GlueArgs glue)
{
    const PairParams<T> p = *params_dev;
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* wbase = smem_raw + warp * FM_WARP_BYTES;
    uint2* meta = reinterpret_cast<uint2*>(wbase);
    unsigned short* list = reinterpret_cast<unsigned short*>(wbase + FM_META * 8);
    int* delta = reinterpret_cast<int*>(wbase + FM_META * 8 + FM_META * 2);
    uint32_t* flags = reinterpret_cast<uint32_t*>(delta + 32);
    const uint32_t le = lanemask_lt() | (1u << (threadIdx.x & 31));

    const DevHeader* hp = p.h;
    if (hp->status & RG_FATAL) return;
    const int nx = hp->nx, ny = hp->ny, nz = hp->nz, S = hp->group_cells, Sy = hp->group_cells_y, pad = hp->pad;
    const uint32_t gx = (uint32_t)hp->gx;
    const uint32_t gy = (uint32_t)((ny + Sy - 1) / Sy);
    const uint32_t num_groups = p.glist ? hp->active_groups : (uint32_t)hp->num_groups;
    const int Wd = 2 * pad + 1, Wy = Sy + 2 * pad, nrun = Wy * Wd;
    const int lane_dy = (lane % Wy) - pad, lane_dz = (lane / Wy) - pad;
    const uint32_t lt = lanemask_lt();

    // target ranges and source run of a group; the next group's are requested while the current group
    // is written, so that one round trip to memory per group (the candidate records) stays exposed
    struct GroupDesc { uint32_t tb0, te0, tb1, te1; int run_a, run_len; };
    auto fetch = [&](uint32_t gi) -> GroupDesc {
        GroupDesc d;
        const uint32_t grp = p.glist ? p.glist[gi] : gi;
        const uint32_t row = grp / gx;
        const int ix = (int)(grp - row * gx);
        const int cz = (int)(row / gy), iy = (int)(row - (uint32_t)cz * gy);
        const int cx0 = ix * S, cx1 = min(cx0 + S, nx) - 1;
        const int cy0 = iy * Sy, cy1 = min(cy0 + Sy, ny) - 1;
        d.tb0 = p.tcstart[((uint32_t)cz * ny + cy0) * nx + cx0];
        d.te0 = p.tcstart[((uint32_t)cz * ny + cy0) * nx + cx1 + 1];
        d.tb1 = d.te1 = 0;
        if (cy1 > cy0) {
            d.tb1 = p.tcstart[((uint32_t)cz * ny + cy1) * nx + cx0];
            d.te1 = p.tcstart[((uint32_t)cz * ny + cy1) * nx + cx1 + 1];
        }
        d.run_a = 0;
        d.run_len = 0;
        if (lane < nrun) {
            const int yy = cy0 + lane_dy, zz = cz + lane_dz;
            if (yy >= 0 && yy < ny && yy <= cy1 + pad && zz >= 0 && zz < nz) {
                const uint32_t b = ((uint32_t)zz * ny + yy) * nx;
                const uint32_t a = p.cstart[b + max(cx0 - pad, 0)];
                const uint32_t e = p.cstart[b + min(cx1 + pad, nx - 1) + 1];
                d.run_a = (int)a;
                d.run_len = (int)(e - a);
            }
        }
        return d;
    };

    const uint32_t nwarps = gridDim.x * PAIR_WARPS;
    uint32_t grp = blockIdx.x * PAIR_WARPS + warp;
    if (grp >= num_groups) return;
    GroupDesc nd = fetch(grp);
    for (; grp < num_groups; grp += nwarps) {
        const GroupDesc d = nd;
        if (grp + nwarps < num_groups) nd = fetch(grp + nwarps);
        uint32_t tb[2] = {d.tb0, d.tb1}, te[2] = {d.te0, d.te1};
        if (tb[0] == te[0] && tb[1] == te[1]) continue;
        const int run_a = d.run_a, run_len = d.run_len;
        // the first target's words do not depend on the candidate records: ask for them now
        int4 ntm;
        long long nbase;
        uint32_t nw;
        {
            const uint32_t t = tb[0] != te[0] ? tb[0] : tb[1];
            ntm = p.tmeta[t]; nbase = p.toffset[t]; nw = p.hitmask[(size_t)t * 32 + lane];
        }
        int L;
        const int run_off = warp_excl_scan(run_len, lane, &L);
        const int nslots = (L + 31) >> 5;
        if (nslots == 0 || nslots > RG_MASK_SLOTS) continue;  // a longer list has no hit bits: rg_pair_kernel<FILL> writes that group

        __syncwarp();
        runs_compact(delta, run_a, run_off, run_len, lt);
        int rank_base = runs_flags(flags, run_off, run_len, lane, 0);
        // four slots at a time: the four gathers are in flight together before the first is stored (measured
        // against asynchronous 8-byte copies into shared memory: equal on sparse cells, faster on dense ones)
        for (int sw0 = 0; sw0 < nslots; sw0 += 4) {
            uint2 mv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int sw = sw0 + u, j = sw * 32 + lane;
                const uint32_t word = (sw < nslots) ? flags[sw] : 0u;
                const int r = rank_base + __popc(word & le) - 1;
                rank_base += __popc(word);
                mv[u] = (j < L) ? p.smeta[delta[r] + j] : make_uint2(0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = (sw0 + u) * 32 + lane;
                if (j < L) meta[j] = mv[u];
            }
        }
        __syncwarp();

        // Targets of both rows as one list, one at a time; the words of the next target are requested
        // before the current one is written.  Lane l holds the hit bits of candidates l, 32 + l, ...:
        // a warp scan of the bit counts gives every lane the place of its first edge, so the edges of a
        // target are ordered by (candidate mod 32, candidate / 32).
        const int n0 = (int)(te[0] - tb[0]), nT = n0 + (int)(te[1] - tb[1]);
        for (int q = 0; q < nT; q++) {
            const int4 tm = ntm;
            const long long base = nbase;
            uint32_t w = nw;
            if (q + 1 < nT) {
                const int qa = q + 1;
                const uint32_t t = qa < n0 ? tb[0] + qa : tb[1] + (qa - n0);
                ntm = p.tmeta[t]; nbase = p.toffset[t]; nw = p.hitmask[(size_t)t * 32 + lane];
            }
            int cnt;
            int pos = warp_excl_scan(__popc(w), lane, &cnt);
            __syncwarp();
            while (w) {
                const int sbit = __ffs((int)w) - 1;
                w &= w - 1;
                list[pos++] = (unsigned short)(sbit * 32 + lane);
            }
            __syncwarp();
            const int sx = tm.y - 512, sy = tm.z - 512, sz = tm.w - 512;
            const long long dst_id = (GLUE && glue.id_map) ? glue.id_map[tm.x] : (long long)tm.x;
            for (int i = lane; i < cnt; i += 32) {
                const uint2 m = meta[list[i]];
                const uint32_t code = m.y;
                const long long e = base + i;
                ei[e] = (GLUE && glue.id_map) ? glue.id_map[m.x] : (long long)m.x;
                ei[E + e] = dst_id;
                if (GLUE) {
                    glue_write(glue, shifts, e, (int)(code & 1023u) + sx, (int)((code >> 10) & 1023u) + sy, (int)((code >> 20) & 1023u) + sz);
                } else {
                    shifts[3 * e + 0] = (float)((int)(code & 1023u) + sx);
                    shifts[3 * e + 1] = (float)((int)((code >> 10) & 1023u) + sy);
                    shifts[3 * e + 2] = (float)((int)((code >> 20) & 1023u) + sz);
                }
            }
        }
    }
}

// First launch of a plan: the header block (it travels as a kernel argument: no staging copy of a pageable host
// buffer), the cell counters, the degree counters and the caller's degree array in one pass.
struct HeaderBlock { uint32_t words[RG_HEADER_BYTES / 4]; };
__global__ void __launch_bounds__(256)
rg_init_kernel(uint32_t* __restrict__ hdr, const HeaderBlock blk, uint4* __restrict__ zero_a, int64_t n_a16,
               uint4* __restrict__ zero_b, int64_t n_b16, int32_t* __restrict__ counts_out, int64_t Nt)
{
    const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    if (i0 < RG_HEADER_BYTES / 4) hdr[i0] = blk.words[i0];
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int64_t i = i0; i < n_a16; i += stride) zero_a[i] = z;
    for (int64_t i = i0; i < n_b16; i += stride) zero_b[i] = z;
    if (counts_out != nullptr)
        for (int64_t i = i0; i < Nt; i += stride) counts_out[i] = 0;
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int pair_grid_waves() { return PAIR_GRID_WAVES; }

struct RgLayout {
    int64_t hdr, partials, tpartials, posw, aff, ccount, cfill, tccount, tcfill, srec, spos, sxyz, scode, smeta, hitmask, trec, tpos, tmeta,
        tcount, toffset, sums, total;
};

static RgLayout rg_layout(int64_t N, int64_t Nt, int64_t src_cap, int64_t cell_cap, int dtype)
{
    const int64_t v4 = dtype == DYNB_F64 ? 32 : 16;
    RgLayout L;
    int64_t o = 0;
    auto take = [&](int64_t bytes) { int64_t r = o; o = align_up(o + bytes, 256); return r; };
    L.hdr = take(RG_HEADER_BYTES);
    // zero-initialised block: cell counters (contiguous so that one memset clears them)
    L.ccount = take((cell_cap + 2) * 4);
    L.cfill = take((cell_cap + 2) * 4);
    L.tccount = take((cell_cap + 2) * 4);
    L.tcfill = take((cell_cap + 2) * 4);
    L.partials = take(((N + 255) / 256 + 1) * 64);
    L.tpartials = take(((Nt + 255) / 256 + 1) * 64);
    L.posw = take(N * v4);
    L.aff = take(N * 16);
    L.srec = take(src_cap * 16);  // {key, cell} of every source image, in slot order
    L.spos = take(src_cap * v4);
    L.sxyz = take(dtype == DYNB_F64 ? 0 : src_cap * 12);  // fp32 only: x[], y[], z[] of the source records for the count pass
    L.scode = take(src_cap * 4);
    L.smeta = take(src_cap * 8);
    L.hitmask = take(Nt * 32 * 2);
    L.trec = take(Nt * 8);        // {entry, cell} of every target, in slot order
    L.tpos = take(Nt * v4);
    L.tmeta = take(Nt * 16);
    L.tcount = take((Nt + 1) * 4);
    L.toffset = take((Nt + 2) * 8);
    const int64_t tiles = std::max<int64_t>(scan_num_tiles(cell_cap + 2), scan_num_tiles(Nt + 2)) + 1;
    L.sums = take(tiles * 8 * 2);
    L.total = o;
    return L;
}

// Host cell geometry in the precision of the positions, following the reference's host code
// (radius_graph_kernels.cu:516-587): face distances, replication counts, cutoff fractions and
// the cofactor inverse.  This translation unit is compiled with -ffp-contract=off for the host.
template <typename T>
static void rg_geometry(const T* cell, const uint8_t* pbc, T radius, Geom<T>& g)
{
    const T* a0 = cell; const T* a1 = cell + 3; const T* a2 = cell + 6;
    T c12[3] = {a1[1] * a2[2] - a1[2] * a2[1], a1[2] * a2[0] - a1[0] * a2[2], a1[0] * a2[1] - a1[1] * a2[0]};
    T vol = a0[0] * c12[0] + a0[1] * c12[1] + a0[2] * c12[2];
    T abs_vol = std::abs(vol);
    T c20[3] = {a2[1] * a0[2] - a2[2] * a0[1], a2[2] * a0[0] - a2[0] * a0[2], a2[0] * a0[1] - a2[1] * a0[0]};
    T c01[3] = {a0[1] * a1[2] - a0[2] * a1[1], a0[2] * a1[0] - a0[0] * a1[2], a0[0] * a1[1] - a0[1] * a1[0]};
    T n12 = std::sqrt(c12[0] * c12[0] + c12[1] * c12[1] + c12[2] * c12[2]);
    T n20 = std::sqrt(c20[0] * c20[0] + c20[1] * c20[1] + c20[2] * c20[2]);
    T n01 = std::sqrt(c01[0] * c01[0] + c01[1] * c01[1] + c01[2] * c01[2]);
    T d_face[3] = {abs_vol / n12, abs_vol / n20, abs_vol / n01};
    for (int d = 0; d < 3; d++) {
        g.pbc[d] = pbc[d] ? 1 : 0;
        if (pbc[d]) {
            g.rep[d] = (int)std::ceil(radius / d_face[d]);
            g.cf[d] = radius / d_face[d];
        } else {
            g.rep[d] = 0;
            g.cf[d] = (T)0;
        }
    }
    T inv_vol = (T)1 / vol;
    g.inv[0] = (a1[1] * a2[2] - a1[2] * a2[1]) * inv_vol;
    g.inv[1] = (a0[2] * a2[1] - a0[1] * a2[2]) * inv_vol;
    g.inv[2] = (a0[1] * a1[2] - a0[2] * a1[1]) * inv_vol;
    g.inv[3] = (a1[2] * a2[0] - a1[0] * a2[2]) * inv_vol;
    g.inv[4] = (a0[0] * a2[2] - a0[2] * a2[0]) * inv_vol;
    g.inv[5] = (a0[2] * a1[0] - a0[0] * a1[2]) * inv_vol;
    g.inv[6] = (a1[0] * a2[1] - a1[1] * a2[0]) * inv_vol;
    g.inv[7] = (a0[1] * a2[0] - a0[0] * a2[1]) * inv_vol;
    g.inv[8] = (a0[0] * a1[1] - a0[1] * a1[0]) * inv_vol;
    for (int i = 0; i < 9; i++) g.cell[i] = cell[i];
}

template <typename T>
static int rg_geometry_checked(const void* cell_host, const uint8_t* pbc_host, double radius, Geom<T>& g)
{
    if (cell_host == nullptr || pbc_host == nullptr) return fail_arg("cell and pbc must not be null");
    if (!(radius > 0.0)) return fail_arg("radius must be positive");
    rg_geometry<T>(static_cast<const T*>(cell_host), pbc_host, (T)radius, g);
    for (int d = 0; d < 3; d++) {
        if (!(g.rep[d] >= 0 && g.rep[d] <= 64) || !std::isfinite((double)g.cf[d]))
            return fail_arg("degenerate cell: a periodic axis needs more than 64 image layers (or the cell is singular)");
    }
    for (int i = 0; i < 9; i++)
        if (!std::isfinite((double)g.inv[i])) return fail_arg("cell matrix is singular");
    return DYNB_OK;
}

template <typename T>
static int rg_suggest(int64_t N, const void* cell_host, const uint8_t* pbc_host, double radius, int64_t* src_cap,
                      int64_t* cell_cap)
{
    Geom<T> g;
    int rc = rg_geometry_checked<T>(cell_host, pbc_host, radius, g);
    if (rc) return rc;
    double full = 1.0, est = 1.0, ext[3] = {0, 0, 0};
    for (int d = 0; d < 3; d++) {
        double span = 1.0;
        if (g.pbc[d]) {
            full *= 2 * g.rep[d] + 1;
            const double reach = g.rep[d] == 1 ? std::min(1.0, (double)g.cf[d]) : (double)g.rep[d];
            est *= 1.0 + 2.0 * reach;
            span = 1.0 + 2.0 * reach;
        }
        for (int k = 0; k < 3; k++) ext[k] += std::fabs((double)g.cell[3 * d + k]) * span;
    }
    const double nmax = (double)N * full;
    double cap = std::min(nmax, (double)N * est * 1.25 + 4096.0);
    if (cap < 1.0) cap = 1.0;
    *src_cap = (int64_t)cap;
    const double res = radius / 1.99;
    double cells = 1.0;
    for (int k = 0; k < 3; k++) cells *= std::ceil((ext[k] + 0.02) / res) + 1.0;
    double ccap = std::min(cells * 1.02 + 64.0, std::max(8.0 * cap, 1048576.0));
    ccap = std::min(ccap, 268435456.0);
    *cell_cap = (int64_t)ccap;
    return DYNB_OK;
}

template <typename T>
static int rg_plan(const void* pos_dev, int64_t N, const void* cell_host, const uint8_t* pbc_host, double radius,
                   const int64_t* targets, int64_t Nt, void* ws, int64_t ws_bytes, int64_t src_cap, int64_t cell_cap,
                   int32_t* counts_out, dynb_rg_header* header_host, cudaStream_t stream)
{
    Geom<T> g;
    int rc = rg_geometry_checked<T>(cell_host, pbc_host, radius, g);
    if (rc) return rc;
    const int dtype = sizeof(T) == 8 ? DYNB_F64 : DYNB_F32;
    const RgLayout L = rg_layout(N, Nt, src_cap, cell_cap, dtype);
    if (ws_bytes < L.total) return fail_arg("workspace too small (see dynb_rg_workspace_bytes)");
    unsigned char* w = static_cast<unsigned char*>(ws);
    DevHeader* h = reinterpret_cast<DevHeader*>(w + L.hdr);

    auto* posw = reinterpret_cast<Vec4<T>*>(w + L.posw);
    auto* aff = reinterpret_cast<int4*>(w + L.aff);
    auto* ccount = reinterpret_cast<uint32_t*>(w + L.ccount);
    auto* cfill = reinterpret_cast<uint32_t*>(w + L.cfill);
    auto* tccount = reinterpret_cast<uint32_t*>(w + L.tccount);
    auto* tcfill = reinterpret_cast<uint32_t*>(w + L.tcfill);
    auto* srec = reinterpret_cast<uint4*>(w + L.srec);
    auto* spos = reinterpret_cast<Vec4<T>*>(w + L.spos);
    float* sxyz = (sizeof(T) == 4) ? reinterpret_cast<float*>(w + L.sxyz) : nullptr;
    auto* scode = reinterpret_cast<uint32_t*>(w + L.scode);
    auto* smeta = reinterpret_cast<uint2*>(w + L.smeta);
    auto* hitmask = reinterpret_cast<unsigned short*>(w + L.hitmask);
    auto* trec = reinterpret_cast<uint2*>(w + L.trec);
    auto* tpos = reinterpret_cast<Vec4<T>*>(w + L.tpos);
    auto* tmeta = reinterpret_cast<int4*>(w + L.tmeta);
    auto* tcount = reinterpret_cast<uint32_t*>(w + L.tcount);
    auto* toffset = reinterpret_cast<long long*>(w + L.toffset);
    auto* sums32 = reinterpret_cast<uint32_t*>(w + L.sums);
    auto* sums64 = reinterpret_cast<long long*>(w + L.sums);
    auto* params_dev = reinterpret_cast<PairParams<T>*>(w + L.hdr + RG_PARAMS_OFFSET);

    static_assert(sizeof(DevHeader) <= RG_PARAMS_OFFSET, "header overlaps params");
    static_assert(RG_PARAMS_OFFSET + sizeof(PairParams<T>) <= RG_HEADER_BYTES, "params overflow header block");
    unsigned char init[RG_HEADER_BYTES];
    memset(init, 0, sizeof(init));
    PairParams<T> pp_host;
    memset(&pp_host, 0, sizeof(pp_host));
    // Periodic in all directions and every atom a target: the images fill a box that follows from the cell alone
    // (fractional coordinates in [1 - cf - rep, cf + rep] per axis, see rg_wrap_kernel's flags), so the grid is
    // chosen here and the first pass counts the images into their cells while it wraps.  Positions that rounding
    // leaves a hair outside land in the outermost cells (cell_of clamps), which a scan window always includes.
    GridChoice gc_host;
    memset(&gc_host, 0, sizeof(gc_host));
    bool host_grid = (targets == nullptr) && g.pbc[0] && g.pbc[1] && g.pbc[2];
    if (host_grid) {
        double lo[3] = {0, 0, 0}, hi3[3] = {0, 0, 0};
        for (int d = 0; d < 3; d++) {
            const double fa = std::max(-(double)g.rep[d], std::min(0.0, 1.0 - (double)g.cf[d] - (double)g.rep[d]));
            const double fb = std::min(1.0 + (double)g.rep[d], std::max(1.0, (double)g.cf[d] + (double)g.rep[d]));
            for (int k = 0; k < 3; k++) {
                const double c = (double)g.cell[3 * d + k];
                lo[k] += std::min(fa * c, fb * c);
                hi3[k] += std::max(fa * c, fb * c);
            }
        }
        double ext[3];
        for (int k = 0; k < 3; k++) {
            const double slack = 0.01 + 1e-5 * (hi3[k] - lo[k]);
            lo[k] -= slack;
            ext[k] = hi3[k] + slack - lo[k];
        }
        const double* c = nullptr;
        double cd[9];
        for (int k = 0; k < 9; k++) cd[k] = (double)g.cell[k];
        c = cd;
        const double vol = std::fabs(c[0] * (c[4] * c[8] - c[5] * c[7]) - c[1] * (c[3] * c[8] - c[5] * c[6]) + c[2] * (c[3] * c[7] - c[4] * c[6]));
        const double density = vol > 0.0 ? (double)N / vol : 0.0;  // images repeat the atoms: the same density everywhere in the box
        rg_choose_grid(lo, ext, radius, (long long)cell_cap, PAIR_CAND_BYTES / (int)sizeof(Vec4<T>), (double)N, density, 0, 0, true, gc_host);
        // A grid over the whole cell that had to take coarser cells to fit the cell capacity (few atoms in a large
        // periodic box) is worse than the grid over the data's own bounding box: that case keeps the device path.
        if (gc_host.res_inv < 0.999 * 1.99 / radius) host_grid = false;
    }
    {
        DevHeader hi;
        memset(&hi, 0, sizeof(hi));
        for (int k = 0; k < 3; k++) { hi.bb_min[k] = ~0ull; hi.bb_max[k] = 0ull; }
        if (host_grid) {
            rg_store_grid(hi, gc_host);
            for (int k = 0; k < 3; k++) { hi.clip_lo[k] = -1.0e300; hi.clip_hi[k] = 1.0e300; }
        }
        memcpy(init, &hi, sizeof(hi));
        PairParams<T>& pp = pp_host;
        pp.h = h; pp.cstart = ccount; pp.tcstart = tccount; pp.spos = spos; pp.sxyz = sxyz; pp.sxyz_stride = src_cap; pp.scode = scode; pp.smeta = smeta; pp.hitmask = hitmask; pp.counts_out = counts_out; pp.tpos = tpos;
        pp.tmeta = tmeta; pp.tcount = tcount; pp.toffset = toffset; pp.r2 = (T)radius * (T)radius;
        // the targets' fill counters are free once the targets are binned: they hold the list of groups with targets
        pp.glist = (targets != nullptr) ? tcfill : nullptr;
        pp.long_list = cfill;   // likewise free once the sources are binned
        memcpy(init + RG_PARAMS_OFFSET, &pp, sizeof(pp));
    }
    {
        HeaderBlock blk;
        memcpy(blk.words, init, sizeof(init));
        // every region of the layout starts on a 256-byte boundary and is padded to one
        const int64_t n_a16 = (L.partials - L.ccount) / 16, n_b16 = ((Nt + 1) * 4 + 15) / 16;
        rg_init_kernel<<<sm_count_cached() * 4, 256, 0, stream>>>(reinterpret_cast<uint32_t*>(w + L.hdr), blk,
                                                                  reinterpret_cast<uint4*>(w + L.ccount), n_a16,
                                                                  reinterpret_cast<uint4*>(w + L.tcount), n_b16, counts_out, Nt);
    }

    const int vec_ok = (reinterpret_cast<uintptr_t>(pos_dev) % 16 == 0) ? 1 : 0;
    const int force_sx = 0, force_sy = 0;  // cells per warp work item: chosen by rg_choose_grid
    const int64_t nb = std::max(N, Nt);
    if (host_grid) {
        rg_wrap_kernel<T, true><<<(unsigned)((N + WRAP_THREADS - 1) / WRAP_THREADS), WRAP_THREADS, 0, stream>>>(
            static_cast<const T*>(pos_dev), N, g, vec_ok, posw, aff, h, nullptr, gc_host, ccount, tccount);
    } else {
        rg_wrap_kernel<T, false><<<(unsigned)((N + WRAP_THREADS - 1) / WRAP_THREADS), WRAP_THREADS, 0, stream>>>(
            static_cast<const T*>(pos_dev), N, g, vec_ok, posw, aff, h, reinterpret_cast<unsigned long long*>(w + L.partials), gc_host,
            nullptr, nullptr);
        int n_tpart = 0;
        if (targets != nullptr) {
            n_tpart = (int)((Nt + 255) / 256);
            rg_target_bbox_kernel<T><<<n_tpart, 256, 0, stream>>>(targets, Nt, N, posw, reinterpret_cast<unsigned long long*>(w + L.tpartials));
        }
        rg_grid_kernel<T><<<1, 1024, 0, stream>>>(h, radius, (long long)src_cap, (long long)cell_cap,
                                                 PAIR_CAND_BYTES / (int)sizeof(Vec4<T>), force_sx, force_sy,
                                                 reinterpret_cast<const unsigned long long*>(w + L.partials),
                                                 (int)((N + WRAP_THREADS - 1) / WRAP_THREADS),
                                                 reinterpret_cast<const unsigned long long*>(w + L.tpartials), n_tpart);
        rg_bin_kernel<T, false><<<(unsigned)((nb + 255) / 256), 256, 0, stream>>>(
            N, Nt, targets, g, posw, h, ccount, cfill, tccount, tcfill, srec, trec, (long long)src_cap, 0);
    }
    // cell starts of sources and targets in the same two launches (which also set the fill cursors); the total of the source counts is the
    // number of source images actually binned (<= the count of rg_wrap when clipping): it becomes header.M
    DYNB_CUDA_OK((exclusive_scan_pair<uint32_t, uint32_t>(ccount, ccount, reinterpret_cast<uint32_t*>(&h->M), tccount, tccount, nullptr,
                                                           &h->ncell_plus1, cell_cap + 1, sums32, stream, cfill, tcfill)));
    rg_bin_kernel<T, true><<<(unsigned)((nb + 255) / 256), 256, 0, stream>>>(
        N, Nt, targets, g, posw, h, ccount, cfill, tccount, tcfill, srec, trec, (long long)src_cap,
        host_grid ? PAIR_CAND_BYTES / (int)sizeof(Vec4<T>) : 0);
    const int64_t nf = std::max(src_cap, Nt);
    rg_bin_finalize_kernel<T><<<(unsigned)((nf + 255) / 256), 256, 0, stream>>>(
        N, Nt, targets, g, posw, aff, h, ccount, tccount, srec, trec, spos, sxyz, src_cap, scode, smeta, tpos, tmeta);

    if (targets != nullptr)
        rg_group_list_kernel<T><<<sm_count_cached() * 8, 256, 0, stream>>>(params_dev, tcfill);
    const int smem = PAIR_WARPS * PAIR_WARP_BYTES;
    DYNB_CUDA_OK(cudaFuncSetAttribute(rg_pair_kernel<T, MODE_COUNT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int grid = sm_count_cached() * 4 * pair_grid_waves();
    rg_pair_kernel<T, MODE_COUNT, true><<<grid, PAIR_THREADS, smem, stream>>>(params_dev, pp_host, nullptr, nullptr, nullptr, 0, HaloArgs{}, 0, GlueArgs{});
    DYNB_CUDA_OK((exclusive_scan<uint32_t, long long>(tcount, toffset, nullptr, Nt + 1, sums64,
                                                       reinterpret_cast<long long*>(&h->E), stream)));
    DYNB_CUDA_OK(cudaGetLastError());
    if (header_host != nullptr)
        DYNB_CUDA_OK(cudaMemcpyAsync(header_host, h, sizeof(dynb_rg_header), cudaMemcpyDeviceToHost, stream));
    return DYNB_OK;
}

template <typename T>
static int rg_fill(const void* ws, int64_t* ei, float* shifts, void* d2out, int64_t E, const GlueArgs* glue_opt, cudaStream_t stream)
{
    const unsigned char* w = static_cast<const unsigned char*>(ws);
    const auto* params_dev = reinterpret_cast<const PairParams<T>*>(w + RG_PARAMS_OFFSET);
    const int smem = PAIR_WARPS * PAIR_WARP_BYTES;
    DYNB_CUDA_OK(cudaFuncSetAttribute(rg_pair_kernel<T, MODE_FILL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int grid = sm_count_cached() * 4 * pair_grid_waves();
    GlueArgs glue{};
    if (glue_opt != nullptr) glue = *glue_opt;
    // Without distances the edges come from the hit masks of the counting pass; the groups whose candidate
    // list was too long for the masks (listed on the device by the counting pass; usually none) are written
    // by the distance-recomputing pass behind it.
    const int use_masks = (d2out == nullptr) ? 1 : 0;
    if (use_masks) {
        const int fsmem = PAIR_WARPS * FM_WARP_BYTES;
        if (glue_opt != nullptr) {
            DYNB_CUDA_OK(cudaFuncSetAttribute(rg_fillmask_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fsmem));
            rg_fillmask_kernel<T, true><<<grid, PAIR_THREADS, fsmem, stream>>>(params_dev, reinterpret_cast<long long*>(ei), shifts, (long long)E, glue);
        } else {
            DYNB_CUDA_OK(cudaFuncSetAttribute(rg_fillmask_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, fsmem));
            rg_fillmask_kernel<T, false><<<grid, PAIR_THREADS, fsmem, stream>>>(params_dev, reinterpret_cast<long long*>(ei), shifts, (long long)E, glue);
        }
    }
    // behind the bit-driven writer this launch only has the listed long groups to do (usually none): two waves keep its cost low
    const int fgrid = use_masks ? sm_count_cached() * 4 * std::min(2, pair_grid_waves()) : grid;
    rg_pair_kernel<T, MODE_FILL, false><<<fgrid, PAIR_THREADS, smem, stream>>>(
        params_dev, PairParams<T>{}, reinterpret_cast<long long*>(ei), shifts, static_cast<T*>(d2out), (long long)E, HaloArgs{}, use_masks, glue);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

template <typename T>
static int rg_halo_mark(const void* ws, const HaloArgs& ha, cudaStream_t stream)
{
    const unsigned char* w = static_cast<const unsigned char*>(ws);
    const auto* params_dev = reinterpret_cast<const PairParams<T>*>(w + RG_PARAMS_OFFSET);
    const int smem = PAIR_WARPS * PAIR_WARP_BYTES;
    DYNB_CUDA_OK(cudaFuncSetAttribute(rg_pair_kernel<T, MODE_HALO, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int grid = sm_count_cached() * 4 * pair_grid_waves();
    rg_pair_kernel<T, MODE_HALO, false><<<grid, PAIR_THREADS, smem, stream>>>(params_dev, PairParams<T>{}, nullptr, nullptr, nullptr, 0, ha, 0, GlueArgs{});
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

}  // namespace dynb

// ------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------
using namespace dynb;

extern "C" int dynb_rg_suggest_capacity(int64_t n_atoms, const void* cell_host, const uint8_t* pbc_host, double radius,
                                        int dtype, int64_t* src_capacity, int64_t* cell_capacity)
{
    if (n_atoms < 0 || src_capacity == nullptr || cell_capacity == nullptr) return fail_arg("bad arguments");
    if (dtype == DYNB_F32) return rg_suggest<float>(n_atoms, cell_host, pbc_host, radius, src_capacity, cell_capacity);
    if (dtype == DYNB_F64) return rg_suggest<double>(n_atoms, cell_host, pbc_host, radius, src_capacity, cell_capacity);
    return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
}

extern "C" int dynb_rg_workspace_bytes(int64_t n_atoms, int64_t n_targets, int64_t src_capacity, int64_t cell_capacity,
                                       int dtype, int64_t* bytes)
{
    if (n_atoms < 0 || n_targets < 0 || src_capacity < 1 || cell_capacity < 1 || bytes == nullptr)
        return fail_arg("bad arguments");
    if (dtype != DYNB_F32 && dtype != DYNB_F64) return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
    if (n_atoms >= (1ll << 31) || src_capacity >= (1ll << 31) || n_targets >= (1ll << 31) || cell_capacity >= (1ll << 31) - 8)
        return fail_arg("sizes must stay below 2^31");
    *bytes = rg_layout(n_atoms, n_targets, src_capacity, cell_capacity, dtype).total;
    return DYNB_OK;
}

extern "C" int dynb_rg_plan(const void* pos_dev, int dtype, int64_t n_atoms, const void* cell_host,
                            const uint8_t* pbc_host, double radius, const int64_t* target_indices_dev,
                            int64_t n_targets, void* workspace_dev, int64_t workspace_bytes, int64_t src_capacity,
                            int64_t cell_capacity, int32_t* neighbor_counts_dev, dynb_rg_header* header_host,
                            void* stream)
{
    if (n_atoms <= 0 || n_targets <= 0) return fail_arg("n_atoms and n_targets must be positive (handle empty input in the caller)");
    if (pos_dev == nullptr || workspace_dev == nullptr) return fail_arg("null device pointer");
    if (target_indices_dev == nullptr && n_targets != n_atoms) return fail_arg("n_targets must equal n_atoms without target_indices");
    if (src_capacity < 1 || cell_capacity < 1) return fail_arg("capacities must be positive");
    if (n_atoms >= (1ll << 31) || src_capacity >= (1ll << 31) || n_targets >= (1ll << 31) || cell_capacity >= (1ll << 31) - 8)
        return fail_arg("sizes must stay below 2^31");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DYNB_F32)
        return rg_plan<float>(pos_dev, n_atoms, cell_host, pbc_host, radius, target_indices_dev, n_targets, workspace_dev,
                              workspace_bytes, src_capacity, cell_capacity, neighbor_counts_dev, header_host, s);
    if (dtype == DYNB_F64)
        return rg_plan<double>(pos_dev, n_atoms, cell_host, pbc_host, radius, target_indices_dev, n_targets, workspace_dev,
                               workspace_bytes, src_capacity, cell_capacity, neighbor_counts_dev, header_host, s);
    return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
}

extern "C" int dynb_rg_fill(const void* workspace_dev, int dtype, int64_t* edge_index_dev, float* cell_shifts_dev,
                            void* dist_sq_dev, int64_t E, void* stream)
{
    if (workspace_dev == nullptr) return fail_arg("null workspace");
    if (E < 0) return fail_arg("E must be non-negative");
    if (E == 0) return DYNB_OK;
    if (edge_index_dev == nullptr || cell_shifts_dev == nullptr) return fail_arg("null output pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DYNB_F32) return rg_fill<float>(workspace_dev, edge_index_dev, cell_shifts_dev, dist_sq_dev, E, nullptr, s);
    if (dtype == DYNB_F64) return rg_fill<double>(workspace_dev, edge_index_dev, cell_shifts_dev, dist_sq_dev, E, nullptr, s);
    return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
}

extern "C" int dynb_rg_fill_glue(const void* workspace_dev, int dtype, int64_t* edge_index_dev, float* unit_shifts_dev,
                                 float* cart_shifts_dev, const float* cell_host, int negate_shifts, const int64_t* id_map_dev,
                                 int64_t E, void* stream)
{
    if (workspace_dev == nullptr) return fail_arg("null workspace");
    if (E < 0) return fail_arg("E must be non-negative");
    if (negate_shifts != 0 && negate_shifts != 1) return fail_arg("negate_shifts must be 0 or 1");
    if (cart_shifts_dev != nullptr && cell_host == nullptr) return fail_arg("cell_host is required with cart_shifts_dev");
    if (E == 0) return DYNB_OK;
    if (edge_index_dev == nullptr || unit_shifts_dev == nullptr) return fail_arg("null output pointer");
    GlueArgs g{};
    g.cart = cart_shifts_dev;
    g.id_map = reinterpret_cast<const long long*>(id_map_dev);
    g.negate = negate_shifts;
    for (int k = 0; k < 9; k++) g.c[k] = cell_host != nullptr ? cell_host[k] : 0.0f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DYNB_F32) return rg_fill<float>(workspace_dev, edge_index_dev, unit_shifts_dev, nullptr, E, &g, s);
    if (dtype == DYNB_F64) return rg_fill<double>(workspace_dev, edge_index_dev, unit_shifts_dev, nullptr, E, &g, s);
    return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
}

extern "C" int dynb_rg_halo_mark(const void* workspace_dev, int dtype, const int64_t* owner_dev, int64_t n_atoms,
                                 int64_t world_size, uint32_t* needed_dev, uint8_t* has_foreign_dev, void* stream)
{
    if (workspace_dev == nullptr || owner_dev == nullptr || needed_dev == nullptr || has_foreign_dev == nullptr)
        return fail_arg("null pointer");
    if (n_atoms <= 0 || world_size < 1) return fail_arg("bad sizes");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    HaloArgs ha;
    ha.owner = reinterpret_cast<const long long*>(owner_dev);
    ha.needed = needed_dev;
    ha.has_foreign = has_foreign_dev;
    ha.words = (int)((world_size + 31) / 32);
    DYNB_CUDA_OK(cudaMemsetAsync(needed_dev, 0, (size_t)n_atoms * ha.words * 4, s));
    DYNB_CUDA_OK(cudaMemsetAsync(has_foreign_dev, 0, (size_t)n_atoms, s));
    if (dtype == DYNB_F32) return rg_halo_mark<float>(workspace_dev, ha, s);
    if (dtype == DYNB_F64) return rg_halo_mark<double>(workspace_dev, ha, s);
    return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
}
