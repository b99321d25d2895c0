// Space-filling-curve partition for B200 (sm_100a): bounds -> keys -> contiguous split into W ranks,
// either through a stable LSD radix sort (when the curve-order permutation is wanted) or, for the labels
// alone, through a digit-by-digit selection of the W - 1 split points (no sort).
//
// Replaces sfc_partition_cuda_impl (dynamis_state/src/csrc/partition/sfc_kernels.cu:178-251) and
// its kernels (:32-173).  The key arithmetic (IEEE division by the range, truncating quantisation,
// 21-bit Morton interleave, the 7-iteration bit transform the reference calls "Hilbert") is kept
// expression for expression; the sort is ours: a stable least-significant-digit radix sort on
// 8-bit digits of (key, atom index) pairs, so that atoms with equal keys keep ascending index order
// (the reference's at::sort leaves that order unspecified).

#include "common.cuh"
#include "scan.cuh"
#include "select.cuh"

namespace dynb {

// ------------------------------------------------------------------------------------------ bounds
struct SfcBounds {
    uint32_t mn[3];  // ordered-integer images
    uint32_t mx[3];
    float pmin[3];
    float prange[3];
};

// The 3 * 256 floats of a block's 256 atoms, fetched with 16-byte loads when the array allows it (the rows are
// 12 bytes apart: four atoms share three vectors) and handed to the threads through shared memory.
__device__ __forceinline__ void stage_positions(const float* __restrict__ pos, int64_t n, int64_t block_base, int vec_ok, float* stage)
{
    const int64_t nblock = min((int64_t)256, n - block_base);
    const float* src = pos + block_base * 3;
    if (vec_ok && nblock == 256) {
        const float4* src4 = reinterpret_cast<const float4*>(src);
        float4* dst4 = reinterpret_cast<float4*>(stage);
        if (threadIdx.x < 192) dst4[threadIdx.x] = src4[threadIdx.x];
    } else {
        for (int k = threadIdx.x; k < (int)nblock * 3; k += 256) stage[k] = src[k];
    }
}

__global__ void __launch_bounds__(256)
sfc_minmax_kernel(const float* __restrict__ pos, int64_t n, int vec_ok, SfcBounds* __restrict__ b)
{
    __shared__ __align__(16) float stage[768];
    uint32_t mn[3] = {0xffffffffu, 0xffffffffu, 0xffffffffu}, mx[3] = {0u, 0u, 0u};
    for (int64_t base = (int64_t)blockIdx.x * 256; base < n; base += (int64_t)gridDim.x * 256) {
        __syncthreads();
        stage_positions(pos, n, base, vec_ok, stage);
        __syncthreads();
        if (base + threadIdx.x < n) {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const uint32_t o = ordered_u32(stage[threadIdx.x * 3 + k]);
                mn[k] = min(mn[k], o);
                mx[k] = max(mx[k], o);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < 3; k++) {
            mn[k] = min(mn[k], __shfl_xor_sync(0xffffffffu, mn[k], o));
            mx[k] = max(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
        }
    __shared__ uint32_t red[6][8];
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int k = 0; k < 3; k++) { red[k][threadIdx.x >> 5] = mn[k]; red[3 + k][threadIdx.x >> 5] = mx[k]; }
    }
    __syncthreads();
    if (threadIdx.x < 6) {  // one atomic per block and bound, not one per warp
        uint32_t v = red[threadIdx.x][0];
        for (int w = 1; w < 8; w++) v = (threadIdx.x < 3) ? min(v, red[threadIdx.x][w]) : max(v, red[threadIdx.x][w]);
        if (threadIdx.x < 3) atomicMin(&b->mn[threadIdx.x], v);
        else atomicMax(&b->mx[threadIdx.x - 3], v);
    }
}

// lower bound and range of axis k from the ordered-integer extrema (sfc_kernels.cu:197-198); every
// thread of the key kernel derives them itself, which saves a one-thread launch in between
__device__ __forceinline__ void sfc_axis(const SfcBounds* __restrict__ b, int k, float* lo_out, float* range_out)
{
    const float lo = unordered_f32(b->mn[k]), hi = unordered_f32(b->mx[k]);
    const float range = hi - lo;
    *lo_out = lo;
    *range_out = (range > 0.0f) ? range : 1.0f;
}

// ------------------------------------------------------------------------------------------ keys
__device__ __forceinline__ uint64_t spread_bits_21(uint32_t v)
{
    uint64_t x = v & 0x1FFFFF;
    x = (x | (x << 32)) & 0x1F00000000FFFFULL;
    x = (x | (x << 16)) & 0x1F0000FF0000FFULL;
    x = (x | (x << 8)) & 0x100F00F00F00F00FULL;
    x = (x | (x << 4)) & 0x10C30C30C30C30C3ULL;
    x = (x | (x << 2)) & 0x1249249249249249ULL;
    return x;
}

template <int CURVE>
__global__ void __launch_bounds__(256)
sfc_keys_kernel(const float* __restrict__ pos, int64_t n, int vec_ok, const SfcBounds* __restrict__ b,
                uint64_t* __restrict__ keys, uint32_t* __restrict__ idx)
{
    __shared__ __align__(16) float stage[768];
    const int64_t base = (int64_t)blockIdx.x * 256;
    stage_positions(pos, n, base, vec_ok, stage);
    __syncthreads();
    const int64_t i = base + threadIdx.x;
    if (i >= n) return;
    float lo0, lo1, lo2, rg0, rg1, rg2;
    sfc_axis(b, 0, &lo0, &rg0);
    sfc_axis(b, 1, &lo1, &rg1);
    sfc_axis(b, 2, &lo2, &rg2);
    const float nx = (stage[threadIdx.x * 3 + 0] - lo0) / rg0;
    const float ny = (stage[threadIdx.x * 3 + 1] - lo1) / rg1;
    const float nz = (stage[threadIdx.x * 3 + 2] - lo2) / rg2;
    uint64_t key;
    if (CURVE == 0) {
        const uint32_t grid_max = (1u << 21) - 1;
        const uint32_t ix = min((uint32_t)(nx * grid_max), grid_max);
        const uint32_t iy = min((uint32_t)(ny * grid_max), grid_max);
        const uint32_t iz = min((uint32_t)(nz * grid_max), grid_max);
        key = spread_bits_21(ix) | (spread_bits_21(iy) << 1) | (spread_bits_21(iz) << 2);
    } else {
        const int order = 7;
        const int grid_max = (1 << order) - 1;
        const int x = min(max((int)(nx * grid_max), 0), grid_max);
        const int y = min(max((int)(ny * grid_max), 0), grid_max);
        const int z = min(max((int)(nz * grid_max), 0), grid_max);
        long long result = 0;
#pragma unroll
        for (int bit = 0; bit < order; bit++) {
            const int xb = (x >> bit) & 1, yb = (y >> bit) & 1, zb = (z >> bit) & 1;
            int nxb, nyb, nzb;
            if (bit == 0) {
                nxb = xb; nyb = yb; nzb = zb;
            } else {
                nxb = xb ? zb : xb;
                nyb = xb ? yb : (yb ? zb : yb);
                nzb = xb ? yb : (yb ? xb : (zb ? yb : zb));
            }
            result |= ((long long)nxb << (3 * bit)) | ((long long)nyb << (3 * bit + 1)) | ((long long)nzb << (3 * bit + 2));
        }
        key = (uint64_t)result;
    }
    keys[i] = key;
    if (idx != nullptr) idx[i] = (uint32_t)i;
}

// ------------------------------------------------------------------------------------------ radix sort
constexpr int RS_THREADS = 256;
constexpr int RS_ITEMS = 4;  // 1024 keys per block: enough blocks to fill the GPU at 1 M keys
constexpr int RS_TILE = RS_THREADS * RS_ITEMS;
constexpr int RS_WARPS = RS_THREADS / 32;

__global__ void __launch_bounds__(RS_THREADS)
rs_hist_kernel(const uint64_t* __restrict__ keys, int64_t n, int shift, int nblocks, uint32_t* __restrict__ ghist)
{
    __shared__ uint32_t hist[256];
    hist[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * RS_TILE;
#pragma unroll
    for (int i = 0; i < RS_ITEMS; i++) {
        const int64_t j = base + i * RS_THREADS + threadIdx.x;
        if (j < n) atomicAdd(&hist[(uint32_t)(keys[j] >> shift) & 255u], 1u);
    }
    __syncthreads();
    ghist[(int64_t)threadIdx.x * nblocks + blockIdx.x] = hist[threadIdx.x];
}

// Stable scatter: tile order = memory order.  Round i of the tile covers elements
// [i*256, (i+1)*256); within a round a warp covers 32 consecutive elements.  The rank of an
// element among equal digits of the tile = (count in earlier rounds and earlier warps of its
// round) + (count among lower lanes of its warp), the latter from __match_any_sync.
__global__ void __launch_bounds__(RS_THREADS)
rs_scatter_kernel(const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                  uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n, int shift, int nblocks,
                  const uint32_t* __restrict__ goffset)
{
    __shared__ uint16_t cnt[RS_ITEMS][RS_WARPS][256];
    __shared__ uint32_t dbase[256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < RS_ITEMS * RS_WARPS * 256; k += RS_THREADS) (&cnt[0][0][0])[k] = 0;
    __syncthreads();

    const int64_t base = (int64_t)blockIdx.x * RS_TILE;
    uint64_t key[RS_ITEMS];
    uint32_t val[RS_ITEMS];
    uint16_t rank[RS_ITEMS];
    const uint32_t lt = lanemask_lt();
#pragma unroll
    for (int i = 0; i < RS_ITEMS; i++) {
        const int64_t j = base + i * RS_THREADS + threadIdx.x;
        const bool live = j < n;
        key[i] = live ? keys_in[j] : ~0ull;
        val[i] = live ? vals_in[j] : 0u;
        const uint32_t d = (uint32_t)(key[i] >> shift) & 255u;
        // dead lanes vote with an impossible digit so that they never join a live group
        const uint32_t peers = __match_any_sync(0xffffffffu, live ? d : 256u + lane);
        rank[i] = (uint16_t)__popc(peers & lt);
        if (live && (peers & lt) == 0) cnt[i][warp][d] = (uint16_t)__popc(peers);
    }
    __syncthreads();
    {
        const int d = threadIdx.x;
        uint32_t run = 0;
#pragma unroll
        for (int i = 0; i < RS_ITEMS; i++)
#pragma unroll
            for (int w = 0; w < RS_WARPS; w++) {
                const uint32_t c = cnt[i][w][d];
                cnt[i][w][d] = (uint16_t)run;
                run += c;
            }
        dbase[d] = goffset[(int64_t)d * nblocks + blockIdx.x];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RS_ITEMS; i++) {
        const int64_t j = base + i * RS_THREADS + threadIdx.x;
        if (j < n) {
            const uint32_t d = (uint32_t)(key[i] >> shift) & 255u;
            const int64_t p = (int64_t)dbase[d] + cnt[i][warp][d] + rank[i];
            keys_out[p] = key[i];
            vals_out[p] = val[i];
        }
    }
}

static inline int rs_num_blocks(int64_t n) { return (int)((n + RS_TILE - 1) / RS_TILE); }

struct RsLayout { int64_t keys_b, vals_b, ghist, sums, total; };
static RsLayout rs_layout(int64_t n)
{
    RsLayout L;
    int64_t o = 0;
    auto take = [&](int64_t b) { int64_t r = o; o = align_up(o + b, 256); return r; };
    const int nb = rs_num_blocks(n);
    L.keys_b = take(n * 8);
    L.vals_b = take(n * 4);
    L.ghist = take((int64_t)nb * 256 * 4 + 64);
    L.sums = take((int64_t)(scan_num_tiles((int64_t)nb * 256) + 1) * 8);
    L.total = o;
    return L;
}

// Sorts (keys, vals) by bits [begin_bit, end_bit) of the keys.  Result ends in keys/vals (the
// caller's arrays): an odd number of passes is finished with a copy.
static int rs_sort_pairs(uint64_t* keys, uint32_t* vals, int64_t n, int begin_bit, int end_bit, unsigned char* ws,
                         cudaStream_t stream)
{
    if (n <= 0) return DYNB_OK;
    const RsLayout L = rs_layout(n);
    uint64_t* kb = reinterpret_cast<uint64_t*>(ws + L.keys_b);
    uint32_t* vb = reinterpret_cast<uint32_t*>(ws + L.vals_b);
    uint32_t* ghist = reinterpret_cast<uint32_t*>(ws + L.ghist);
    uint32_t* sums = reinterpret_cast<uint32_t*>(ws + L.sums);
    const int nb = rs_num_blocks(n);
    uint64_t* kin = keys; uint32_t* vin = vals; uint64_t* kout = kb; uint32_t* vout = vb;
    for (int shift = begin_bit; shift < end_bit; shift += 8) {
        rs_hist_kernel<<<nb, RS_THREADS, 0, stream>>>(kin, n, shift, nb, ghist);
        DYNB_CUDA_OK((exclusive_scan<uint32_t, uint32_t>(ghist, ghist, nullptr, (int64_t)nb * 256, sums, nullptr, stream)));
        rs_scatter_kernel<<<nb, RS_THREADS, 0, stream>>>(kin, vin, kout, vout, n, shift, nb, ghist);
        std::swap(kin, kout);
        std::swap(vin, vout);
    }
    if (kin != keys) {
        DYNB_CUDA_OK(cudaMemcpyAsync(keys, kin, (size_t)n * 8, cudaMemcpyDeviceToDevice, stream));
        DYNB_CUDA_OK(cudaMemcpyAsync(vals, vin, (size_t)n * 4, cudaMemcpyDeviceToDevice, stream));
    }
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

// ------------------------------------------------------------------------------------------ assignment
__global__ void __launch_bounds__(256)
sfc_assign_unweighted_kernel(const uint32_t* __restrict__ perm, int64_t* __restrict__ labels, int64_t N, int64_t W)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int64_t base = N / W, rem = N % W, threshold = rem * (base + 1);  // sfc_kernels.cu:123-134
    int64_t p;
    if (i < threshold) p = i / (base + 1);
    else p = rem + (i - threshold) / base;
    p = min(p, W - 1);
    labels[perm[i]] = p;
}

__global__ void __launch_bounds__(256)
sfc_gather_weights_kernel(const int64_t* __restrict__ w, const uint32_t* __restrict__ perm, int64_t* __restrict__ sorted_w, int64_t N)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) sorted_w[i] = w[perm[i]];
}

// excl[i] = sum of sorted weights before i; the reference uses the inclusive sum (:165-170)
__global__ void __launch_bounds__(256)
sfc_assign_weighted_kernel(const uint32_t* __restrict__ perm, const int64_t* __restrict__ sorted_w,
                           const int64_t* __restrict__ excl, const int64_t* __restrict__ total_p,
                           int64_t* __restrict__ labels, int64_t N, int64_t W)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int64_t total = *total_p;
    const int64_t cs = excl[i] + sorted_w[i];
    int64_t p = (total > 0) ? (cs * W) / total : (int64_t)0;
    p = max(p, (int64_t)0);
    p = min(p, W - 1);
    labels[perm[i]] = p;
}

__global__ void __launch_bounds__(256) fill_i64_kernel(int64_t* p, int64_t n, int64_t v)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

__global__ void __launch_bounds__(256) u32_to_i64_kernel(const uint32_t* a, int64_t* b, int64_t n)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) b[i] = (int64_t)a[i];
}


// ------------------------------------------------------------------------------------------ labels by selection
// When only the labels are wanted (no curve-order permutation), the sort is not needed: an atom's
// label is the number of split points at or before it in (key, atom index) order, and the W - 1 split
// points — for label p the first atom, in that order, whose inclusive prefix weight reaches
// ceil(p * total / W) (unit weights: the atom of rank first_rank(p)) — are found by a most-significant-
// digit descent on the composite number C = key << idx_bits | index.  Every level is a weighted digit
// histogram of the atoms that still share a split point's prefix (one pass over the keys, atomics on a
// table in L2) and one block per split point that walks the histogram to the digit where its threshold
// is crossed.  Six levels of 16 bits cover Morton keys of a million atoms: 12 small launches instead
// of the 40 of the eight radix passes, and nothing but the keys is read.
// Weights must be non-negative here (degrees); the labels are those of the sorted path.

// Distinct prefixes of the live split points (they are non-decreasing) into glist (loaded by the whole
// block, compacted in place).  All threads of the block call this; returns the number of groups.
__device__ int sel_groups(const SelSplit* __restrict__ st, int nsplit, u128* glist, int* gid_of_split)
{
    __shared__ int s_ng;
    __shared__ int s_live;
    if (threadIdx.x == 0) s_live = nsplit;
    __syncthreads();
    for (int s = threadIdx.x; s < nsplit; s += blockDim.x) {
        const SelSplit v = st[s];
        glist[s] = sel_prefix(v);
        if (v.dead) atomicMin(&s_live, s);  // dead split points are the last ones
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int ng = 0;
        const int live = s_live;
        for (int s = 0; s < live; s++) {
            const u128 p = glist[s];  // ng <= s: the compaction never overtakes the read
            if (ng == 0 || glist[ng - 1] != p) glist[ng++] = p;
            if (gid_of_split) gid_of_split[s] = ng - 1;
        }
        if (gid_of_split)
            for (int s = live; s < nsplit; s++) gid_of_split[s] = -1;
        s_ng = ng;
    }
    __syncthreads();
    return s_ng;
}

// A warp finds, among up to 256 counters at p, the first whose inclusive prefix reaches R: returns its
// index to all lanes (-1 if the sum stays below R), *before = weight in front of it, *total = sum of all.
__device__ int sel_warp_cross(const unsigned long long* p, int count, long long R, long long* before, long long* total)
{
    const int lane = threadIdx.x & 31;
    long long v[8];
    long long local = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int i = lane * 8 + k;
        v[k] = (i < count) ? (long long)__ldcg(p + i) : 0ll;  // counters were written by atomics: read them at L2
        local += v[k];
    }
    long long x = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const long long y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    *total = __shfl_sync(0xffffffffu, x, 31);
    const bool mine = (x - local < R) && (R <= x);
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (m == 0u) return -1;
    int idx = -1;
    long long bef = 0, c = x - local;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        if (idx < 0 && c + v[k] >= R) { idx = lane * 8 + k; bef = c; }
        c += v[k];
    }
    const int src = __ffs((int)m) - 1;
    *before = __shfl_sync(0xffffffffu, bef, src);
    return __shfl_sync(0xffffffffu, idx, src);
}

// One warp advances split point s by one level: coarse counters -> run of digits -> the digit where its
// threshold is crossed.  gid: group of every split point at this level (not read at level 0).
__device__ void sel_pick_warp(int s, const SelSplit* __restrict__ st_in, SelSplit* __restrict__ st_out, const int* gid,
                              int nsplit, int level, int width, int dbits, int64_t n, int64_t W, int weighted,
                              const long long* thresholds, const unsigned long long* hist)
{
    const int lane = threadIdx.x & 31;
    SelSplit me;
    int g = 0;
    if (level == 0) {
        me.pre_hi = me.pre_lo = 0; me.residual = 0; me.dead = 0; me.pad = 0;
    } else {
        me = st_in[s];
        g = gid[s];
        if (me.dead) {
            if (lane == 0) st_out[s] = me;
            return;
        }
    }
    const unsigned long long* fine = hist + ((size_t)g << dbits);
    const unsigned long long* coarse = hist + ((size_t)nsplit << dbits) + ((size_t)g << 8);
    const int fbits = min(width, 8);
    const int nc = 1 << (width - fbits);  // coarse counters in use (<= 256)
    long long R = me.residual;
    long long before_c = 0, before_f = 0, total = 0;
    int cb;
    if (level == 0) {
        // the total first: thresholds of sfc_kernels.cu:123-134 (equal counts) and :165-170 (weights)
        sel_warp_cross(coarse, nc, 0x7fffffffffffffffll, &before_c, &total);
        const long long p = s + 1;
        long long T;
        if (thresholds != nullptr) {
            T = thresholds[s];
        } else if (weighted) {
            T = (total > 0) ? (long long)(((u128)p * (u128)total + (u128)(W - 1)) / (u128)W) : total + 1;
            if (T < 1) T = 1;
        } else {
            const long long base = n / W, rem = n % W;
            const long long first = (p <= rem) ? p * (base + 1) : rem * (base + 1) + (p - rem) * base;
            T = first + 1;
        }
        me.residual = R = T;
        me.dead = (T > total) ? 1 : 0;
        if (me.dead) {
            if (lane == 0) st_out[s] = me;
            return;
        }
    }
    cb = sel_warp_cross(coarse, nc, R, &before_c, &total);
    if (cb < 0) return;  // cannot happen: the threshold lies inside this group
    const int fb = sel_warp_cross(fine + ((size_t)cb << fbits), 1 << fbits, R - before_c, &before_f, &total);
    if (fb < 0) return;
    if (lane == 0) {
        const unsigned digit = ((unsigned)cb << fbits) | (unsigned)fb;
        const u128 P = (sel_prefix(me) << width) | (u128)digit;
        me.pre_hi = (unsigned long long)(P >> 64);
        me.pre_lo = (unsigned long long)P;
        me.residual = R - before_c - before_f;
        st_out[s] = me;
    }
}

// Early finish.  From the second level on the atoms that still share a split point's prefix are few (a million
// Morton keys spread over 2^14 first digits leave a few hundred), so the level's pass also appends them — full
// composite number, weight, group — to a short list, and the block that finishes last settles every split point
// from that list at once: the split atom of a group is the listed atom with the smallest composite number whose
// inclusive prefix weight inside the group reaches the split point's residual.  The remaining levels then return
// at once.  A list that overflows, or a group with more than SEL_FINISH_GROUP_MAX atoms, leaves the level as it
// was and the next level tries again.
struct SelCand { unsigned long long hi, lo; long long w; int g; int pad; };
static_assert(sizeof(SelCand) == sizeof(SelSplit), "candidates share the unused split-point slots");
constexpr int SEL_FINISH_SPLITS = 16;        // the fused path's limit on split points
constexpr int SEL_CAND_CAP = SEL_MAX_SPLITS - SEL_FINISH_SPLITS;   // records behind the split points of state buffer 0
constexpr int SEL_FINISH_GROUP_MAX = 128;

__device__ __forceinline__ SelCand sel_load_cand(const SelCand* p)
{
    const ulonglong2 a = __ldcg(reinterpret_cast<const ulonglong2*>(p));
    const ulonglong2 b = __ldcg(reinterpret_cast<const ulonglong2*>(p) + 1);
    SelCand c;
    c.hi = a.x; c.lo = a.y; c.w = (long long)b.x; c.g = (int)(unsigned)(b.y & 0xffffffffull); c.pad = 0;
    return c;
}

// One warp settles split point s from the candidate list; member[] is the warp's scratch (SEL_FINISH_GROUP_MAX
// entries).  Returns false (to all lanes) if the group is too large or no listed atom reaches the residual.
__device__ bool sel_finish_warp(const SelSplit& me, int g, const SelCand* cand, int total, unsigned short* member, SelSplit* out)
{
    const int lane = threadIdx.x & 31;
    const unsigned lt = lanemask_lt();
    int m = 0;
    for (int base = 0; base < total; base += 32) {
        const int i = base + lane;
        bool in = false;
        if (i < total) in = ((int)(unsigned)(__ldcg(reinterpret_cast<const unsigned long long*>(cand + i) + 3) & 0xffffffffull) == g);
        const unsigned mm = __ballot_sync(0xffffffffu, in);
        if (in) {
            const int at = m + __popc(mm & lt);
            if (at < SEL_FINISH_GROUP_MAX) member[at] = (unsigned short)i;
        }
        m += __popc(mm);
    }
    __syncwarp();
    if (m == 0 || m > SEL_FINISH_GROUP_MAX) return false;
    // every lane takes the members lane, 32 + lane, ... into registers; each member is then handed round by
    // shuffles and added to the inclusive weight of every member that is not smaller: no memory in the loop
    constexpr int KM = SEL_FINISH_GROUP_MAX / 32;
    const int kmax = (m + 31) >> 5;
    unsigned long long chi[KM], clo[KM];
    long long cw[KM], inc[KM];
#pragma unroll
    for (int k = 0; k < KM; k++) {
        chi[k] = clo[k] = ~0ull;
        cw[k] = 0;
        inc[k] = 0;
        const int a = lane + 32 * k;
        if (a < m) {
            const SelCand c = sel_load_cand(cand + member[a]);
            chi[k] = c.hi; clo[k] = c.lo; cw[k] = c.w;
        }
    }
#pragma unroll
    for (int kb = 0; kb < KM; kb++) {
        if (kb < kmax) {
            const int nb = min(32, m - 32 * kb);
            for (int lb = 0; lb < nb; lb++) {
                const unsigned long long bh = __shfl_sync(0xffffffffu, chi[kb], lb), bl = __shfl_sync(0xffffffffu, clo[kb], lb);
                const long long bw = __shfl_sync(0xffffffffu, cw[kb], lb);
#pragma unroll
                for (int ka = 0; ka < KM; ka++)
                    if (ka < kmax && (bh < chi[ka] || (bh == chi[ka] && bl <= clo[ka]))) inc[ka] += bw;
            }
        }
    }
    u128 best = ~(u128)0;
#pragma unroll
    for (int k = 0; k < KM; k++) {
        const u128 Ca = ((u128)chi[k] << 64) | (u128)clo[k];
        if (lane + 32 * k < m && inc[k] >= me.residual && Ca < best) best = Ca;
    }
    unsigned long long bh = (unsigned long long)(best >> 64), bl = (unsigned long long)best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long oh = __shfl_xor_sync(0xffffffffu, bh, o), ol = __shfl_xor_sync(0xffffffffu, bl, o);
        if (oh < bh || (oh == bh && ol < bl)) { bh = oh; bl = ol; }
    }
    if (bh == ~0ull && bl == ~0ull) return false;
    if (lane == 0) {
        SelSplit r = me;
        r.pre_hi = bh; r.pre_lo = bl; r.residual = 0;
        *out = r;
    }
    return true;
}

// Table of one level: per group 2^dbits digit counters ("fine"), followed by per group 256 coarse
// counters, one per run of 2^fbits consecutive digits (fbits = min(width, 8)), so that a split point is
// located by reading 256 + 256 counters instead of the whole digit range.
// With done_counter != nullptr the block that finishes last also advances the split points (one warp
// each), which saves a launch per level; used while there are few split points.
__global__ void __launch_bounds__(256, 4)   // four blocks per SM for the histogram pass; the rare finish may spill
sel_hist_kernel(const uint64_t* __restrict__ keys, const int64_t* __restrict__ weights, int64_t n, int idx_bits,
                int shift, int width, int dbits, const SelSplit* st, SelSplit* __restrict__ st_out, int nsplit,
                int level, int64_t W, const long long* __restrict__ thresholds, unsigned long long* __restrict__ hist,
                unsigned long long* __restrict__ hist_next, int64_t table_words, unsigned int* __restrict__ done_counter,
                int fine_private, SelCand* __restrict__ cand, unsigned int* __restrict__ cand_count,
                unsigned int* __restrict__ finished, SelSplit* st_other /* the buffer st points into: no restrict */)
{
    // fine_private (first level, unit weights, width <= 14 only): the digit counters of this block are kept in
    // shared memory and added to the table once at the end -- for keys that crowd into a few digits (the
    // ordered bits of float coordinates) a million atomics on a handful of addresses took 90-150 us
    extern __shared__ unsigned int s_fine[];
    __shared__ u128 glist[SEL_MAX_SPLITS];
    __shared__ int gid[SEL_MAX_SPLITS];
    __shared__ unsigned long long s_coarse[256];
    __shared__ bool s_last;
    // cand != nullptr: the early finish is in use (see above); finished: set by the level that settled the split points
    if (cand != nullptr && __ldcg(finished) != 0u) return;
    // clear the table the next level accumulates into (its last reader, the previous pick, has finished)
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < table_words; k += (int64_t)gridDim.x * blockDim.x)
        hist_next[k] = 0ull;
    unsigned long long* coarse = hist + ((size_t)nsplit << dbits);
    const int fbits = min(width, 8);
    int ng = 1;
    if (level == 0) {
        if (threadIdx.x == 0) glist[0] = 0;
        s_coarse[threadIdx.x] = 0ull;  // one group, every atom counts: coarse counters through shared memory
        if (fine_private)
            for (int k = threadIdx.x; k < (1 << width); k += blockDim.x) s_fine[k] = 0u;
        __syncthreads();
    } else {
        ng = sel_groups(st, nsplit, glist, gid);
    }
    const u128 dmask = ((u128)1 << width) - 1;
    if (ng > 0) {
        // warp-uniform trip count (all 32 lanes take part in the vote below); lanes past the end carry no counter
        const int64_t warp_base = (int64_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31);
        for (int64_t base = warp_base; base < n; base += (int64_t)gridDim.x * blockDim.x) {
            const int64_t i = base + (threadIdx.x & 31);
            unsigned long long w = 0ull;
            size_t slot = ~(size_t)0;  // counter of this atom, or none
            unsigned digit = 0;
            int lo = 0;
            u128 C = 0;
            if (i < n) {
                C = ((u128)keys[i] << idx_bits) | (u128)(uint64_t)i;
                const u128 P = C >> (shift + width);
                int hi = ng;  // first group with prefix >= P
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (glist[mid] < P) lo = mid + 1; else hi = mid;
                }
                if (lo < ng && glist[lo] == P) {
                    w = weights ? (unsigned long long)weights[i] : 1ull;
                    if (w) {
                        digit = (unsigned)((C >> shift) & dmask);
                        slot = ((size_t)lo << dbits) + digit;
                    }
                }
            }
            if (cand != nullptr && level > 0) {
                // the atoms counted at this level, listed for the early finish (one atomic per warp round)
                const bool listed = (slot != ~(size_t)0);
                const unsigned lm = __ballot_sync(0xffffffffu, listed);
                if (lm) {
                    const int leader = __ffs((int)lm) - 1;
                    unsigned at = 0;
                    if ((int)(threadIdx.x & 31) == leader) at = atomicAdd(cand_count, (unsigned)__popc(lm));
                    at = __shfl_sync(0xffffffffu, at, leader) + (unsigned)__popc(lm & lanemask_lt());
                    if (listed && at < (unsigned)SEL_CAND_CAP) {
                        SelCand c;
                        c.hi = (unsigned long long)(C >> 64); c.lo = (unsigned long long)C; c.w = (long long)w; c.g = lo; c.pad = 0;
                        cand[at] = c;
                    }
                }
            }
            if (fine_private) {
                // crowded keys: lanes that hit the same counter send one atomic between them
                const unsigned peers = __match_any_sync(0xffffffffu, (unsigned long long)slot);
                if (slot != ~(size_t)0 && (threadIdx.x & 31) == __ffs((int)peers) - 1) w = (unsigned long long)__popc(peers);
                else w = 0ull;
            }
            if (w) {
                if (fine_private) atomicAdd(&s_fine[digit], (unsigned int)w);
                else atomicAdd(&hist[slot], w);
                if (level == 0) atomicAdd(&s_coarse[digit >> fbits], w);
                else atomicAdd(&coarse[((size_t)lo << 8) + (digit >> fbits)], w);
            }
        }
    }
    if (level == 0) {
        __syncthreads();
        const unsigned long long v = s_coarse[threadIdx.x];
        if (v) atomicAdd(&coarse[threadIdx.x], v);
        if (fine_private)
            for (int k = threadIdx.x; k < (1 << width); k += blockDim.x) {
                const unsigned int c = s_fine[k];
                if (c) atomicAdd(&hist[k], (unsigned long long)c);
            }
    }
    if (done_counter == nullptr) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int s = threadIdx.x >> 5; s < nsplit; s += (int)(blockDim.x >> 5))
        sel_pick_warp(s, st, st_out, gid, nsplit, level, width, dbits, n, W, weights != nullptr ? 1 : 0, thresholds, hist);
    if (cand == nullptr || level == 0 || nsplit > SEL_FINISH_SPLITS) return;
    // early finish: settle every split point from the list, or leave the level's result as it is
    __shared__ SelSplit s_fin[SEL_FINISH_SPLITS];
    __shared__ unsigned short s_member[8][SEL_FINISH_GROUP_MAX];
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    const int total = (int)__ldcg(cand_count);
    if (total > SEL_CAND_CAP) return;
    for (int s = threadIdx.x >> 5; s < nsplit; s += (int)(blockDim.x >> 5)) {
        const SelSplit me = st[s];
        if (me.dead) {
            if ((threadIdx.x & 31) == 0) s_fin[s] = me;
        } else if (!sel_finish_warp(me, gid[s], cand, total, s_member[threadIdx.x >> 5], &s_fin[s])) {
            if ((threadIdx.x & 31) == 0) s_fail = 1;
        }
    }
    __syncthreads();
    if (s_fail) return;
    // whichever state buffer the caller reads after the last level holds the settled split points
    for (int s = threadIdx.x; s < nsplit; s += blockDim.x) { st_out[s] = s_fin[s]; st_other[s] = s_fin[s]; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *finished = 1u;
}

// the same step as its own launch, eight split points per block (many split points)
__global__ void __launch_bounds__(256)
sel_pick_kernel(const SelSplit* __restrict__ st_in, SelSplit* __restrict__ st_out, int nsplit, int level, int width, int dbits,
                int64_t n, int64_t W, int weighted, const long long* __restrict__ thresholds,
                const unsigned long long* __restrict__ hist)
{
    __shared__ u128 glist[SEL_MAX_SPLITS];
    __shared__ int gid[SEL_MAX_SPLITS];
    if (level > 0) sel_groups(st_in, nsplit, glist, gid);
    const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (s < nsplit) sel_pick_warp(s, st_in, st_out, gid, nsplit, level, width, dbits, n, W, weighted, thresholds, hist);
}

__global__ void __launch_bounds__(256)
sel_label_kernel(const uint64_t* __restrict__ keys, int64_t n, int idx_bits, const SelSplit* __restrict__ st, int nsplit,
                 int64_t* __restrict__ labels)
{
    __shared__ u128 cs[SEL_MAX_SPLITS];
    __shared__ int s_live;
    if (threadIdx.x == 0) s_live = nsplit;
    __syncthreads();
    for (int s = threadIdx.x; s < nsplit; s += blockDim.x) {
        const SelSplit v = st[s];
        cs[s] = sel_prefix(v);
        if (v.dead) atomicMin(&s_live, s);  // dead split points are the last ones
    }
    __syncthreads();
    const int live = s_live;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const u128 C = ((u128)keys[i] << idx_bits) | (u128)(uint64_t)i;
        int lo = 0, hi = live;  // number of split points <= C
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (cs[mid] <= C) lo = mid + 1; else hi = mid;
        }
        labels[i] = (int64_t)lo;
    }
}

// digit width: the widest the table budget allows for W - 1 groups, then narrowed while the number
// of levels stays the same (a narrower digit means a smaller table to clear per level)
static int sel_digit_bits(int64_t groups, int total_bits)
{
    int d = 16;
    while (d > 8 && groups * (((int64_t)8 << d) + 2048) + 256 > SEL_HIST_BYTES) d--;
    const int levels = (total_bits + d - 1) / d;
    while (d > 8 && (total_bits + (d - 1) - 1) / (d - 1) == levels) d--;
    return d;
}

int sel_select_splits(const uint64_t* keys, int key_bits, const int64_t* weights_dev, int64_t n, int nsplit, int64_t W,
                      const long long* thresholds_dev, unsigned char* state_ws, unsigned char* hist_ws, int* idx_bits_out,
                      const SelSplit** final_out, bool crowded_keys, cudaStream_t s)
{
    if (nsplit < 1 || nsplit > SEL_MAX_SPLITS) return fail_arg("number of split points out of range");
    int idx_bits = 1;
    while (idx_bits < 32 && ((int64_t)1 << idx_bits) < n) idx_bits++;
    const int B = key_bits + idx_bits;
    const int dbits = sel_digit_bits(nsplit, B);
    const int levels = (B + dbits - 1) / dbits;
    SelSplit* st = reinterpret_cast<SelSplit*>(state_ws);
    unsigned long long* hist = reinterpret_cast<unsigned long long*>(hist_ws);
    const int64_t hist_words = SEL_HIST_BYTES / 8;
    const int64_t table_words = ((int64_t)nsplit << dbits) + ((int64_t)nsplit << 8);  // digit + coarse counters of a level
    // the first table and, behind it, one arrival counter per level
    unsigned int* counters = reinterpret_cast<unsigned int*>(hist + table_words);
    DYNB_CUDA_OK(cudaMemsetAsync(hist, 0, (size_t)table_words * 8 + 256, s));
    const bool fused = nsplit <= SEL_FINISH_SPLITS;  // two rounds of eight warps in the last block
    // early finish (fused path only): candidates in the split-point slots of state buffer 0 that no level uses,
    // one list counter per level behind the arrival counters, then the "finished" word
    SelCand* cand = fused ? reinterpret_cast<SelCand*>(st + SEL_FINISH_SPLITS) : nullptr;
    unsigned int* cand_counts = counters + 16;
    unsigned int* finished = counters + 48;
    if (levels > 16) return fail_arg("too many digit levels");
    const int hgrid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)sm_count_cached() * 4);  // one wave
    for (int l = 0; l < levels; l++) {
        const int width = std::min(dbits, B - l * dbits);
        const int shift = B - l * dbits - width;
        const SelSplit* st_in = st + (size_t)(l & 1) * SEL_MAX_SPLITS;
        SelSplit* st_out = st + (size_t)((l + 1) & 1) * SEL_MAX_SPLITS;
        unsigned long long* h_cur = hist + (size_t)(l & 1) * hist_words;
        unsigned long long* h_other = hist + (size_t)((l + 1) & 1) * hist_words;
        unsigned int* done = fused ? counters + l : nullptr;
        const int priv = (crowded_keys && l == 0 && weights_dev == nullptr && width <= 14) ? 1 : 0;
        const size_t dyn = priv ? ((size_t)4 << width) : 0;
        // static + dynamic shared memory beyond 48 KB needs the opt-in
        if (dyn > 0) DYNB_CUDA_OK(cudaFuncSetAttribute(sel_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        sel_hist_kernel<<<hgrid, 256, dyn, s>>>(keys, weights_dev, n, idx_bits, shift, width, dbits, st_in, st_out, nsplit, l, W,
                                                thresholds_dev, h_cur, h_other, table_words, done, priv, cand, cand_counts + l, finished,
                                                const_cast<SelSplit*>(st_in));
        if (!fused)
            sel_pick_kernel<<<(nsplit + 7) / 8, 256, 0, s>>>(st_in, st_out, nsplit, l, width, dbits, n, W,
                                                             weights_dev != nullptr ? 1 : 0, thresholds_dev, h_cur);
    }
    DYNB_CUDA_OK(cudaGetLastError());
    *idx_bits_out = idx_bits;
    *final_out = st + (size_t)(levels & 1) * SEL_MAX_SPLITS;
    return DYNB_OK;
}

struct SfcLayout { int64_t bounds, keys, idx, sorted_w, excl, total_w, sums, rs, total_sort, sel_state, sel_hist, total; };
static SfcLayout sfc_layout(int64_t n)
{
    SfcLayout L;
    int64_t o = 0;
    auto take = [&](int64_t b) { int64_t r = o; o = align_up(o + b, 256); return r; };
    L.bounds = take(sizeof(SfcBounds));
    L.keys = take(n * 8);
    L.idx = take(n * 4);
    L.sorted_w = take(n * 8);
    L.excl = take(n * 8);
    L.total_w = take(64);
    L.sums = take((int64_t)(scan_num_tiles(n) + 1) * 8);
    L.rs = take(rs_layout(n).total);
    L.total_sort = o;  // enough for the sorted path
    L.sel_state = take(2 * SEL_MAX_SPLITS * (int64_t)sizeof(SelSplit));
    L.sel_hist = take(2 * SEL_HIST_BYTES);
    L.total = o;
    return L;
}

static int sfc_keys_into(const float* pos, int64_t n, int curve, unsigned char* ws, const SfcLayout& L, uint64_t* keys,
                         uint32_t* idx, cudaStream_t stream)
{
    // extrema start at +max / 0 in the ordered-integer image; set on the device (no copy from host memory)
    SfcBounds* b = reinterpret_cast<SfcBounds*>(ws + L.bounds);
    DYNB_CUDA_OK(cudaMemsetAsync(b->mn, 0xff, sizeof(b->mn), stream));
    DYNB_CUDA_OK(cudaMemsetAsync(b->mx, 0, sizeof(SfcBounds) - sizeof(b->mn), stream));
    const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)sm_count_cached() * 4);
    const int vec_ok = (reinterpret_cast<uintptr_t>(pos) % 16 == 0) ? 1 : 0;
    sfc_minmax_kernel<<<grid, 256, 0, stream>>>(pos, n, vec_ok, b);
    const unsigned nbk = (unsigned)((n + 255) / 256);
    if (curve == 0) sfc_keys_kernel<0><<<nbk, 256, 0, stream>>>(pos, n, vec_ok, b, keys, idx);
    else sfc_keys_kernel<1><<<nbk, 256, 0, stream>>>(pos, n, vec_ok, b, keys, idx);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}


// ------------------------------------------------------------------------------------------ pieces for a partition
// whose atoms are spread over several ranks: bounds as plain floats (to be min/max-reduced between the
// ranks), keys against given bounds, labels from agreed split points
__global__ void sfc_bounds_to_float_kernel(const SfcBounds* __restrict__ b, float* __restrict__ minmax)
{
    if (threadIdx.x < 3) minmax[threadIdx.x] = unordered_f32(b->mn[threadIdx.x]);
    else if (threadIdx.x < 6) minmax[threadIdx.x] = unordered_f32(b->mx[threadIdx.x - 3]);
}

__global__ void sfc_bounds_from_float_kernel(const float* __restrict__ minmax, SfcBounds* __restrict__ b)
{
    if (threadIdx.x < 3) b->mn[threadIdx.x] = ordered_u32(minmax[threadIdx.x]);
    else if (threadIdx.x < 6) b->mx[threadIdx.x - 3] = ordered_u32(minmax[threadIdx.x]);
}

// labels[i] = number of split points (K_s, G_s) <= (keys[i], ids[i]) in lexicographic order; the split
// points are sorted ascending.
__global__ void __launch_bounds__(256)
label_by_splits_kernel(const int64_t* __restrict__ keys, const int64_t* __restrict__ ids, int64_t n,
                       const int64_t* __restrict__ split_keys, const int64_t* __restrict__ split_ids, int nsplit,
                       int64_t* __restrict__ labels)
{
    __shared__ unsigned long long sk[SEL_MAX_SPLITS];
    __shared__ long long sg[SEL_MAX_SPLITS];
    for (int s = threadIdx.x; s < nsplit; s += blockDim.x) { sk[s] = (unsigned long long)split_keys[s]; sg[s] = split_ids[s]; }
    __syncthreads();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const unsigned long long k = (unsigned long long)keys[i];
        const long long g = ids[i];
        int lo = 0, hi = nsplit;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            const bool le = sk[mid] < k || (sk[mid] == k && sg[mid] <= g);
            if (le) lo = mid + 1; else hi = mid;
        }
        labels[i] = lo;
    }
}

}  // namespace dynb

using namespace dynb;

extern "C" int dynb_sfc_workspace_bytes(int64_t n_atoms, int64_t* bytes)
{
    if (n_atoms < 0 || bytes == nullptr || n_atoms >= (1ll << 32) - 1) return fail_arg("bad arguments");
    *bytes = sfc_layout(std::max<int64_t>(n_atoms, 1)).total;
    return DYNB_OK;
}

extern "C" int dynb_sfc_keys(const float* pos_dev, int64_t n_atoms, int curve_type, int64_t* keys_dev, void* workspace_dev,
                             int64_t workspace_bytes, void* stream)
{
    if (n_atoms < 0 || (curve_type != 0 && curve_type != 1)) return fail_arg("curve_type must be 0 (Morton) or 1 (Hilbert)");
    if (n_atoms == 0) return DYNB_OK;
    if (pos_dev == nullptr || keys_dev == nullptr || workspace_dev == nullptr) return fail_arg("null pointer");
    const SfcLayout L = sfc_layout(n_atoms);
    if (workspace_bytes < L.total) return fail_arg("workspace too small (see dynb_sfc_workspace_bytes)");
    return sfc_keys_into(pos_dev, n_atoms, curve_type, static_cast<unsigned char*>(workspace_dev), L,
                         reinterpret_cast<uint64_t*>(keys_dev), nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int dynb_sfc_minmax(const float* pos_dev, int64_t n_atoms, float* minmax_dev, void* stream)
{
    if (n_atoms < 0 || minmax_dev == nullptr) return fail_arg("bad arguments");
    if (n_atoms > 0 && pos_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the 24 bytes behind the six floats are the scratch for the ordered-integer extrema
    SfcBounds* b = reinterpret_cast<SfcBounds*>(minmax_dev + 8);
    DYNB_CUDA_OK(cudaMemsetAsync(b->mn, 0xff, sizeof(b->mn), s));
    DYNB_CUDA_OK(cudaMemsetAsync(b->mx, 0, sizeof(b->mx), s));
    if (n_atoms > 0) {
        const int grid = (int)std::min<int64_t>((n_atoms + 255) / 256, (int64_t)sm_count_cached() * 4);
        sfc_minmax_kernel<<<grid, 256, 0, s>>>(pos_dev, n_atoms, (reinterpret_cast<uintptr_t>(pos_dev) % 16 == 0) ? 1 : 0, b);
    }
    sfc_bounds_to_float_kernel<<<1, 32, 0, s>>>(b, minmax_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_sfc_keys_from_bounds(const float* pos_dev, int64_t n_atoms, int curve_type, float* minmax_dev,
                                         int64_t* keys_dev, void* stream)
{
    if (n_atoms < 0 || (curve_type != 0 && curve_type != 1)) return fail_arg("curve_type must be 0 (Morton) or 1 (Hilbert)");
    if (minmax_dev == nullptr) return fail_arg("null pointer");
    if (n_atoms == 0) return DYNB_OK;
    if (pos_dev == nullptr || keys_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    SfcBounds* b = reinterpret_cast<SfcBounds*>(minmax_dev + 8);
    sfc_bounds_from_float_kernel<<<1, 32, 0, s>>>(minmax_dev, b);
    const unsigned nbk = (unsigned)((n_atoms + 255) / 256);
    const int vec_ok = (reinterpret_cast<uintptr_t>(pos_dev) % 16 == 0) ? 1 : 0;
    if (curve_type == 0) sfc_keys_kernel<0><<<nbk, 256, 0, s>>>(pos_dev, n_atoms, vec_ok, b, reinterpret_cast<uint64_t*>(keys_dev), nullptr);
    else sfc_keys_kernel<1><<<nbk, 256, 0, s>>>(pos_dev, n_atoms, vec_ok, b, reinterpret_cast<uint64_t*>(keys_dev), nullptr);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_label_by_splits(const int64_t* keys_dev, const int64_t* ids_dev, int64_t n, const int64_t* split_keys_dev,
                                    const int64_t* split_ids_dev, int n_splits, int64_t* labels_dev, void* stream)
{
    if (n < 0 || n_splits < 0 || n_splits > SEL_MAX_SPLITS) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    if (keys_dev == nullptr || ids_dev == nullptr || labels_dev == nullptr || (n_splits > 0 && (split_keys_dev == nullptr || split_ids_dev == nullptr)))
        return fail_arg("null pointer");
    const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)sm_count_cached() * 8);
    label_by_splits_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(keys_dev, ids_dev, n, split_keys_dev, split_ids_dev,
                                                                             n_splits, labels_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_sfc_partition(const float* pos_dev, int64_t n_atoms, const int64_t* weights_dev, int64_t W, int curve_type,
                                  int64_t* labels_dev, int64_t* perm_dev, void* workspace_dev, int64_t workspace_bytes,
                                  void* stream)
{
    if (n_atoms < 0) return fail_arg("n_atoms must be non-negative");
    if (W < 1) return fail_arg("W must be >= 1");
    if (curve_type != 0 && curve_type != 1) return fail_arg("curve_type must be 0 (Morton) or 1 (Hilbert)");
    if (n_atoms == 0) return DYNB_OK;
    if (pos_dev == nullptr || labels_dev == nullptr || workspace_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned nbk = (unsigned)((n_atoms + 255) / 256);
    if (W == 1 && perm_dev == nullptr) {  // sfc_kernels.cu:192-194
        fill_i64_kernel<<<nbk, 256, 0, s>>>(labels_dev, n_atoms, 0);
        DYNB_CUDA_OK(cudaGetLastError());
        return DYNB_OK;
    }
    const SfcLayout L = sfc_layout(n_atoms);
    if (workspace_bytes < L.total_sort) return fail_arg("workspace too small (see dynb_sfc_workspace_bytes)");
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    uint64_t* keys = reinterpret_cast<uint64_t*>(ws + L.keys);
    uint32_t* idx = reinterpret_cast<uint32_t*>(ws + L.idx);
    if (perm_dev == nullptr && W >= 2 && W - 1 <= SEL_MAX_SPLITS && workspace_bytes >= L.total) {
        // labels by selection (no sort)
        int rc = sfc_keys_into(pos_dev, n_atoms, curve_type, ws, L, keys, nullptr, s);
        if (rc) return rc;
        const int nsplit = (int)(W - 1);
        int idx_bits = 0;
        const SelSplit* splits = nullptr;
        rc = sel_select_splits(keys, curve_type == 0 ? 63 : 21, weights_dev, n_atoms, nsplit, W, nullptr, ws + L.sel_state, ws + L.sel_hist,
                               &idx_bits, &splits, false, s);
        if (rc) return rc;
        const int hgrid = (int)std::min<int64_t>((n_atoms + 255) / 256, (int64_t)sm_count_cached() * 4);
        sel_label_kernel<<<hgrid, 256, 0, s>>>(keys, n_atoms, idx_bits, splits, nsplit, labels_dev);
        DYNB_CUDA_OK(cudaGetLastError());
        return DYNB_OK;
    }
    int rc = sfc_keys_into(pos_dev, n_atoms, curve_type, ws, L, keys, idx, s);
    if (rc) return rc;
    rc = rs_sort_pairs(keys, idx, n_atoms, 0, curve_type == 0 ? 64 : 24, ws + L.rs, s);
    if (rc) return rc;
    if (W == 1) {
        fill_i64_kernel<<<nbk, 256, 0, s>>>(labels_dev, n_atoms, 0);
    } else if (weights_dev != nullptr) {
        int64_t* sorted_w = reinterpret_cast<int64_t*>(ws + L.sorted_w);
        int64_t* excl = reinterpret_cast<int64_t*>(ws + L.excl);
        int64_t* total = reinterpret_cast<int64_t*>(ws + L.total_w);
        sfc_gather_weights_kernel<<<nbk, 256, 0, s>>>(weights_dev, idx, sorted_w, n_atoms);
        DYNB_CUDA_OK((exclusive_scan<long long, long long>(reinterpret_cast<long long*>(sorted_w), reinterpret_cast<long long*>(excl),
                                                            nullptr, n_atoms, reinterpret_cast<long long*>(ws + L.sums),
                                                            reinterpret_cast<long long*>(total), s)));
        sfc_assign_weighted_kernel<<<nbk, 256, 0, s>>>(idx, sorted_w, excl, total, labels_dev, n_atoms, W);
    } else {
        sfc_assign_unweighted_kernel<<<nbk, 256, 0, s>>>(idx, labels_dev, n_atoms, W);
    }
    if (perm_dev != nullptr) u32_to_i64_kernel<<<nbk, 256, 0, s>>>(idx, perm_dev, n_atoms);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_radix_sort_workspace_bytes(int64_t n, int64_t* bytes)
{
    if (n < 0 || bytes == nullptr) return fail_arg("bad arguments");
    *bytes = rs_layout(std::max<int64_t>(n, 1)).total;
    return DYNB_OK;
}

extern "C" int dynb_radix_sort_pairs(uint64_t* keys_dev, uint32_t* vals_dev, int64_t n, int begin_bit, int end_bit,
                                     void* workspace_dev, int64_t workspace_bytes, void* stream)
{
    if (n < 0 || begin_bit < 0 || end_bit > 64 || begin_bit >= end_bit || (begin_bit % 8) != 0)
        return fail_arg("bad bit range (begin_bit must be a multiple of 8, end_bit <= 64)");
    if (n == 0) return DYNB_OK;
    if (keys_dev == nullptr || vals_dev == nullptr || workspace_dev == nullptr) return fail_arg("null pointer");
    if (workspace_bytes < rs_layout(n).total) return fail_arg("workspace too small");
    return rs_sort_pairs(keys_dev, vals_dev, n, begin_bit, end_bit, static_cast<unsigned char*>(workspace_dev),
                         static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------ no-allocation variant
// Some hosts of this library may not allocate device memory at all while they run: an MD engine that
// hands its whole memory budget to its own pool at start-up, a plugin living inside another runtime's
// allocator, a latency-critical loop where a cudaMalloc (which synchronises the device) is not
// acceptable.  They cannot provide the workspace dynb_sfc_partition asks for.  This variant keeps that
// workspace in a fixed device array that is part of the library image, so every GPU that loads the
// library carries DYNB_SFC_STATIC_BYTES of it until the process exits, and problems larger than
// DYNB_SFC_STATIC_MAX_ATOMS are refused.
constexpr int64_t DYNB_SFC_STATIC_MAX_ATOMS_C = 131072;
constexpr int64_t DYNB_SFC_STATIC_BYTES = 6ll << 20;
static __device__ __align__(256) unsigned char g_sfc_static_scratch[DYNB_SFC_STATIC_BYTES];
// Device address of the array, per device.  In host code the array's name is only a stand-in and
// must never be handed to a kernel; cudaGetSymbolAddress gives the real address for the current device.
static void* g_sfc_static_addr[64] = {nullptr};

extern "C" int64_t dynb_sfc_static_max_atoms(void) { return DYNB_SFC_STATIC_MAX_ATOMS_C; }

extern "C" int dynb_sfc_partition_static(const float* pos_dev, int64_t n_atoms, const int64_t* weights_dev, int64_t W,
                                         int curve_type, int64_t* labels_dev, int64_t* perm_dev, void* stream)
{
    if (n_atoms < 0) return dynb::fail_arg("n_atoms must be non-negative");
    if (n_atoms > DYNB_SFC_STATIC_MAX_ATOMS_C)
        return dynb::fail_arg("dynb_sfc_partition_static: n_atoms exceeds the built-in scratch (limit 131072 atoms); "
                              "use dynb_sfc_partition with a caller-provided workspace");
    if (dynb::sfc_layout(std::max<int64_t>(n_atoms, 1)).total_sort > DYNB_SFC_STATIC_BYTES)
        return dynb::fail_arg("dynb_sfc_partition_static: built-in scratch too small for this size");
    int dev = 0;
    DYNB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return dynb::fail_arg("device ordinal out of range");
    if (g_sfc_static_addr[dev] == nullptr) {
        void* p = nullptr;
        DYNB_CUDA_OK(cudaGetSymbolAddress(&p, g_sfc_static_scratch));
        if (p == nullptr) return dynb::fail_arg("cudaGetSymbolAddress returned a null address");
        g_sfc_static_addr[dev] = p;
    }
    return dynb_sfc_partition(pos_dev, n_atoms, weights_dev, W, curve_type, labels_dev, perm_dev, g_sfc_static_addr[dev],
                              DYNB_SFC_STATIC_BYTES, stream);
}
