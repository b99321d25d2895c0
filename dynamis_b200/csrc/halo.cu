// Partition bookkeeping and halo-map assembly for B200 (sm_100a).
//
//   dynb_bincount_i64 / dynb_select_eq_i64   atom_counts and partition_indices of
//       SFCPartitioner::do_partition (dynamis_state/src/csrc/partition/sfc_partitioner.cpp:166-176)
//   dynb_halo_mark_from_edges                per-edge pass of extract_halo_info
//       (dynamis_state/src/csrc/graph/dist_graph_ops_kernels.cu:46-59, 104-188)
//   dynb_csr_plan / dynb_csr_fill            send / recv CSR of build_halo_maps
//       (dynamis_state/src/csrc/build_halo_maps.cpp:60-125) and of extract_halo_info, from a
//       per-atom rank bit mask instead of the reference's [N, W] bool matrix + nonzero + argsort
//   dynb_filter_edges_plan / _fill           filter_edges_to_radius
//       (dist_graph_ops_kernels.cu:16-43, 62-102)
//
// Every list these produce is in the reference's order: grouped by peer rank ascending, inside a
// peer ascending atom id.  That order falls out of a stable per-peer compaction over atoms in
// ascending id, so nothing is sorted.

#include "common.cuh"
#include "scan.cuh"

namespace dynb {

// ------------------------------------------------------------------------------------------ bincount / select
__global__ void __launch_bounds__(256)
bincount_i64_kernel(const int64_t* __restrict__ a, int64_t n, int64_t W, unsigned long long* __restrict__ counts,
                    uint32_t* __restrict__ bad)
{
    extern __shared__ uint32_t hist[];
    const bool use_smem = W <= 4096;
    if (use_smem) {
        for (int k = threadIdx.x; k < W; k += blockDim.x) hist[k] = 0;
        __syncthreads();
    }
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = a[i];
        if (v < 0 || v >= W) { atomicOr(bad, 1u); continue; }
        if (use_smem) atomicAdd(&hist[v], 1u);
        else atomicAdd(&counts[v], 1ull);
    }
    if (use_smem) {
        __syncthreads();
        for (int k = threadIdx.x; k < W; k += blockDim.x)
            if (hist[k]) atomicAdd(&counts[k], (unsigned long long)hist[k]);
    }
}

__global__ void __launch_bounds__(256)
flag_eq_i64_kernel(const int64_t* __restrict__ a, int64_t n, int64_t value, uint32_t* __restrict__ flags)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) flags[i] = (a[i] == value) ? 1u : 0u;
}

__global__ void __launch_bounds__(256)
scatter_selected_kernel(const int64_t* __restrict__ a, int64_t n, int64_t value, const uint32_t* __restrict__ excl,
                        const int64_t* __restrict__ gather_src, int64_t* __restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && a[i] == value) out[excl[i]] = gather_src ? gather_src[i] : i;
}

__global__ void u32_total_to_i64_kernel(const uint32_t* t, int64_t* out) { *out = (int64_t)(*t); }

// ------------------------------------------------------------------------------------------ edge marking
// For every edge src -> dst of one rank's edge list (dst owned by my_rank): when the source is
// owned by a peer p, that peer must send src to me (recv side) and I must send dst to p (send
// side, by the symmetry of the radius graph).
__global__ void __launch_bounds__(256)
halo_mark_edges_kernel(const int64_t* __restrict__ src, const int64_t* __restrict__ dst, int64_t E,
                       const int64_t* __restrict__ pid, int64_t N, int64_t my_rank, int words,
                       uint32_t* __restrict__ send_mask, uint32_t* __restrict__ recv_mask,
                       uint8_t* __restrict__ has_remote, uint32_t* __restrict__ bad)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int64_t s = src[e], d = dst[e];
    if (s < 0 || s >= N || d < 0 || d >= N) { atomicOr(bad, 1u); return; }
    const int64_t p = pid[s];
    if (p == my_rank) return;
    if (p < 0 || p >= (int64_t)words * 32) { atomicOr(bad, 2u); return; }
    const uint32_t bit = 1u << (p & 31);
    uint32_t* rw = &recv_mask[s * words + (p >> 5)];
    if (!(*rw & bit)) atomicOr(rw, bit);
    uint32_t* sw = &send_mask[d * words + (p >> 5)];
    if (!(*sw & bit)) atomicOr(sw, bit);
    has_remote[d] = 1;
}

// ------------------------------------------------------------------------------------------ CSR assembly
// Element a in [0, n) carries a set of peer ranks.  For each peer p, the output segment p lists the
// elements whose set contains p, ascending in a.  Modes define the set:
enum { CSR_SEND = 0, CSR_RECV = 1, CSR_RAW = 2 };
//   CSR_SEND  owner[a] == R ? bits of mask[a] without R : {}        (needed_by rows of my atoms)
//   CSR_RECV  owner[a] != R and bit R of mask[a] ? {owner[a]} : {}   (foreign atoms I need)
//   CSR_RAW   bits of mask[a]
constexpr int CSR_THREADS = 256;
constexpr int CSR_WARPS = CSR_THREADS / 32;

__device__ __forceinline__ bool csr_has(const uint32_t* __restrict__ mask, int words, const int64_t* __restrict__ owner,
                                        int64_t a, int64_t R, int mode, int p)
{
    if (mode == CSR_RAW) return (mask[a * words + (p >> 5)] >> (p & 31)) & 1u;
    const int64_t o = owner[a];
    if (mode == CSR_SEND) return o == R && p != R && ((mask[a * words + (p >> 5)] >> (p & 31)) & 1u);
    return o != R && o == p && ((mask[a * words + (R >> 5)] >> (R & 31)) & 1u);
}

// bsum[p * nblocks + block] = number of elements of this block whose set contains p
__global__ void __launch_bounds__(CSR_THREADS)
csr_count_kernel(const uint32_t* __restrict__ mask, int words, const int64_t* __restrict__ owner, int64_t n, int64_t R,
                 int mode, int W, int nblocks, uint32_t* __restrict__ bsum)
{
    __shared__ uint32_t wsum[CSR_WARPS];
    const int64_t a = (int64_t)blockIdx.x * CSR_THREADS + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int p = 0; p < W; p++) {
        const bool f = (a < n) && csr_has(mask, words, owner, a, R, mode, p);
        const uint32_t b = __ballot_sync(0xffffffffu, f);
        if (lane == 0) wsum[warp] = __popc(b);
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t s = 0;
            for (int w = 0; w < CSR_WARPS; w++) s += wsum[w];
            bsum[(int64_t)p * nblocks + blockIdx.x] = s;
        }
        __syncthreads();
    }
}

// One block per peer: exclusive scan of its row of block sums (in place) and the row total.
__global__ void __launch_bounds__(SCAN_THREADS)
csr_scan_rows_kernel(uint32_t* __restrict__ bsum, int nblocks, int64_t* __restrict__ totals)
{
    __shared__ uint32_t warp_sums[SCAN_THREADS / 32];
    uint32_t* row = bsum + (int64_t)blockIdx.x * nblocks;
    uint32_t carry = 0;
    for (int b0 = 0; b0 < nblocks; b0 += SCAN_THREADS) {
        const int i = b0 + threadIdx.x;
        const uint32_t v = (i < nblocks) ? row[i] : 0u;
        uint32_t tot;
        const uint32_t ex = block_excl_scan<uint32_t>(v, &tot, warp_sums);
        if (i < nblocks) row[i] = carry + ex;
        carry += tot;
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = (int64_t)carry;
}

__global__ void csr_offsets_kernel(const int64_t* __restrict__ totals, int W, int64_t* __restrict__ offsets)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int64_t run = 0;
        for (int p = 0; p < W; p++) { offsets[p] = run; run += totals[p]; }
        offsets[W] = run;
    }
}

__global__ void __launch_bounds__(CSR_THREADS)
csr_fill_kernel(const uint32_t* __restrict__ mask, int words, const int64_t* __restrict__ owner, int64_t n, int64_t R,
                int mode, int W, int nblocks, const uint32_t* __restrict__ bsum, const int64_t* __restrict__ offsets,
                const int64_t* __restrict__ value_map, int64_t* __restrict__ out)
{
    __shared__ uint32_t wsum[CSR_WARPS];
    const int64_t a = (int64_t)blockIdx.x * CSR_THREADS + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lt = lanemask_lt();
    for (int p = 0; p < W; p++) {
        const bool f = (a < n) && csr_has(mask, words, owner, a, R, mode, p);
        const uint32_t b = __ballot_sync(0xffffffffu, f);
        if (lane == 0) wsum[warp] = __popc(b);
        __syncthreads();
        if (f) {
            uint32_t before = 0;
            for (int w = 0; w < warp; w++) before += wsum[w];
            const int64_t pos = offsets[p] + bsum[(int64_t)p * nblocks + blockIdx.x] + before + __popc(b & lt);
            out[pos] = value_map ? value_map[a] : a;
        }
        __syncthreads();
    }
}

// local index of each atom inside its owner's ascending list: excl scan of (owner == R)
__global__ void __launch_bounds__(256)
gather_not_u8_kernel(const uint8_t* __restrict__ flags, const int64_t* __restrict__ idx, int64_t n, uint8_t* __restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = flags[idx[i]] ? 0 : 1;
}

__global__ void __launch_bounds__(256)
scatter_iota_kernel(const int64_t* __restrict__ idx, int64_t n, int64_t N, int64_t* __restrict__ g2l, uint32_t* __restrict__ bad)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t a = idx[i];
    if (a < 0 || a >= N) { atomicOr(bad, 4u); return; }
    g2l[a] = i;
}

// ------------------------------------------------------------------------------------------ edge filter
// keep[e] = |pos[src] + shift @ cell - pos[dst]|^2 <= r2, float32, the reference's expression
// (dist_graph_ops_kernels.cu:30-43).
struct Cell9 { float c[9]; };

__global__ void __launch_bounds__(256)
edge_keep_flags_kernel(const int64_t* __restrict__ src, const int64_t* __restrict__ dst, const float* __restrict__ shifts,
                       const float* __restrict__ pos, Cell9 cell, float r2, int64_t E, uint32_t* __restrict__ keep)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int64_t s = src[e];
    const int64_t d = dst[e];
    float sx = pos[3 * s + 0], sy = pos[3 * s + 1], sz = pos[3 * s + 2];
    const float dx = pos[3 * d + 0], dy = pos[3 * d + 1], dz = pos[3 * d + 2];
    const float h0 = shifts[3 * e + 0], h1 = shifts[3 * e + 1], h2 = shifts[3 * e + 2];
    sx += h0 * cell.c[0] + h1 * cell.c[3] + h2 * cell.c[6];
    sy += h0 * cell.c[1] + h1 * cell.c[4] + h2 * cell.c[7];
    sz += h0 * cell.c[2] + h1 * cell.c[5] + h2 * cell.c[8];
    const float ax = sx - dx, ay = sy - dy, az = sz - dz;
    keep[e] = ((ax * ax + ay * ay + az * az) <= r2) ? 1u : 0u;
}

__global__ void __launch_bounds__(256)
edge_compact_kernel(const int64_t* __restrict__ edges, const unsigned char* __restrict__ shifts_raw, int shift_row_bytes,
                    const uint32_t* __restrict__ keep, const uint32_t* __restrict__ excl, int64_t E, int64_t E_out,
                    int64_t* __restrict__ edges_out, unsigned char* __restrict__ shifts_out)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E || !keep[e]) return;
    const int64_t o = excl[e];
    edges_out[o] = edges[e];
    edges_out[E_out + o] = edges[E + e];
    if (shift_row_bytes == 12) {
        const float* a = reinterpret_cast<const float*>(shifts_raw) + 3 * e;
        float* b = reinterpret_cast<float*>(shifts_out) + 3 * o;
        b[0] = a[0]; b[1] = a[1]; b[2] = a[2];
    } else {
        for (int k = 0; k < shift_row_bytes; k++) shifts_out[o * shift_row_bytes + k] = shifts_raw[e * shift_row_bytes + k];
    }
}

static inline unsigned nblk(int64_t n, int t = 256) { return (unsigned)((n + t - 1) / t); }

}  // namespace dynb

using namespace dynb;

// ------------------------------------------------------------------------------------------ C ABI
extern "C" int dynb_bincount_i64(const int64_t* a_dev, int64_t n, int64_t W, int64_t* counts_dev, uint32_t* bad_dev, void* stream)
{
    if (n < 0 || W < 1 || counts_dev == nullptr || bad_dev == nullptr) return fail_arg("bad arguments");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DYNB_CUDA_OK(cudaMemsetAsync(counts_dev, 0, (size_t)W * 8, s));
    DYNB_CUDA_OK(cudaMemsetAsync(bad_dev, 0, 4, s));
    if (n == 0) return DYNB_OK;
    const int grid = (int)std::min<int64_t>(nblk(n), (int64_t)sm_count_cached() * 8);
    const size_t smem = W <= 4096 ? (size_t)W * 4 : 0;
    bincount_i64_kernel<<<grid, 256, smem, s>>>(a_dev, n, W, reinterpret_cast<unsigned long long*>(counts_dev), bad_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_select_workspace_bytes(int64_t n, int64_t* bytes)
{
    if (n < 0 || bytes == nullptr) return fail_arg("bad arguments");
    *bytes = align_up((n + 2) * 4, 256) + align_up((int64_t)(scan_num_tiles(n + 2) + 1) * 8, 256) + 256;
    return DYNB_OK;
}

// out_dev must hold n elements (upper bound); *count_dev receives how many were written.
extern "C" int dynb_select_eq_i64(const int64_t* a_dev, int64_t n, int64_t value, const int64_t* gather_src_dev,
                                  int64_t* out_dev, int64_t* count_dev, void* workspace_dev, int64_t workspace_bytes,
                                  void* stream)
{
    if (n < 0 || count_dev == nullptr) return fail_arg("bad arguments");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n == 0) { DYNB_CUDA_OK(cudaMemsetAsync(count_dev, 0, 8, s)); return DYNB_OK; }
    int64_t need;
    dynb_select_workspace_bytes(n, &need);
    if (workspace_dev == nullptr || workspace_bytes < need) return fail_arg("workspace too small (see dynb_select_workspace_bytes)");
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    uint32_t* flags = reinterpret_cast<uint32_t*>(ws);
    uint32_t* sums = reinterpret_cast<uint32_t*>(ws + align_up((n + 2) * 4, 256));
    uint32_t* total = reinterpret_cast<uint32_t*>(ws + need - 256);
    flag_eq_i64_kernel<<<nblk(n), 256, 0, s>>>(a_dev, n, value, flags);
    DYNB_CUDA_OK((exclusive_scan<uint32_t, uint32_t>(flags, flags, nullptr, n, sums, total, s)));
    scatter_selected_kernel<<<nblk(n), 256, 0, s>>>(a_dev, n, value, flags, gather_src_dev, out_dev);
    u32_total_to_i64_kernel<<<1, 1, 0, s>>>(total, count_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_halo_mark_from_edges(const int64_t* edges_dev, int64_t E, const int64_t* pid_dev, int64_t N, int64_t my_rank,
                                         int64_t world_size, uint32_t* send_mask_dev, uint32_t* recv_mask_dev,
                                         uint8_t* has_remote_dev, uint32_t* bad_dev, void* stream)
{
    if (E < 0 || N < 0 || world_size < 1 || my_rank < 0 || my_rank >= world_size) return fail_arg("bad arguments");
    const int words = (int)((world_size + 31) / 32);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DYNB_CUDA_OK(cudaMemsetAsync(send_mask_dev, 0, (size_t)N * words * 4, s));
    DYNB_CUDA_OK(cudaMemsetAsync(recv_mask_dev, 0, (size_t)N * words * 4, s));
    DYNB_CUDA_OK(cudaMemsetAsync(has_remote_dev, 0, (size_t)N, s));
    DYNB_CUDA_OK(cudaMemsetAsync(bad_dev, 0, 4, s));
    if (E == 0) return DYNB_OK;
    halo_mark_edges_kernel<<<nblk(E), 256, 0, s>>>(edges_dev, edges_dev + E, E, pid_dev, N, my_rank, words, send_mask_dev,
                                                   recv_mask_dev, has_remote_dev, bad_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

static inline int csr_blocks(int64_t n) { return (int)((n + CSR_THREADS - 1) / CSR_THREADS); }

extern "C" int dynb_csr_workspace_bytes(int64_t n, int64_t W, int64_t* bytes)
{
    if (n < 0 || W < 1 || bytes == nullptr) return fail_arg("bad arguments");
    *bytes = align_up((int64_t)std::max(csr_blocks(n), 1) * W * 4, 256) + align_up(W * 8, 256);
    return DYNB_OK;
}

extern "C" int dynb_csr_plan(const uint32_t* mask_dev, const int64_t* owner_dev, int64_t n, int64_t R, int mode, int64_t W,
                             int64_t* offsets_dev, void* workspace_dev, int64_t workspace_bytes, void* stream)
{
    if (n < 0 || W < 1 || mode < 0 || mode > 2 || offsets_dev == nullptr) return fail_arg("bad arguments");
    if (mode != CSR_RAW && owner_dev == nullptr) return fail_arg("owner required");
    if (W > 4096) return fail_arg("world_size above 4096 is not supported");
    int64_t need;
    dynb_csr_workspace_bytes(n, W, &need);
    if (workspace_dev == nullptr || workspace_bytes < need) return fail_arg("workspace too small (see dynb_csr_workspace_bytes)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int words = (int)((W + 31) / 32);
    const int nb = std::max(csr_blocks(n), 1);
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    uint32_t* bsum = reinterpret_cast<uint32_t*>(ws);
    int64_t* totals = reinterpret_cast<int64_t*>(ws + align_up((int64_t)nb * W * 4, 256));
    if (n == 0) {
        DYNB_CUDA_OK(cudaMemsetAsync(offsets_dev, 0, (size_t)(W + 1) * 8, s));
        return DYNB_OK;
    }
    csr_count_kernel<<<nb, CSR_THREADS, 0, s>>>(mask_dev, words, owner_dev, n, R, mode, (int)W, nb, bsum);
    csr_scan_rows_kernel<<<(unsigned)W, SCAN_THREADS, 0, s>>>(bsum, nb, totals);
    csr_offsets_kernel<<<1, 32, 0, s>>>(totals, (int)W, offsets_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_csr_fill(const uint32_t* mask_dev, const int64_t* owner_dev, int64_t n, int64_t R, int mode, int64_t W,
                             const int64_t* value_map_dev, const int64_t* offsets_dev, int64_t* out_dev,
                             const void* workspace_dev, void* stream)
{
    if (n < 0 || W < 1 || mode < 0 || mode > 2) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int words = (int)((W + 31) / 32);
    const int nb = csr_blocks(n);
    const uint32_t* bsum = reinterpret_cast<const uint32_t*>(workspace_dev);
    csr_fill_kernel<<<nb, CSR_THREADS, 0, s>>>(mask_dev, words, owner_dev, n, R, mode, (int)W, nb, bsum, offsets_dev,
                                               value_map_dev, out_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_gather_not_u8(const uint8_t* flags_dev, const int64_t* idx_dev, int64_t n, uint8_t* out_dev, void* stream)
{
    if (n < 0) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    gather_not_u8_kernel<<<nblk(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(flags_dev, idx_dev, n, out_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_scatter_iota(const int64_t* idx_dev, int64_t n, int64_t N, int64_t* g2l_dev, uint32_t* bad_dev, void* stream)
{
    if (n < 0 || N < 0) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    scatter_iota_kernel<<<nblk(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(idx_dev, n, N, g2l_dev, bad_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_filter_edges_plan(const int64_t* edges_dev, const float* shifts_f32_dev, const float* pos_dev,
                                      const float* cell_host, double radius, int64_t E, int64_t* count_dev,
                                      void* workspace_dev, int64_t workspace_bytes, void* stream)
{
    if (E < 0 || count_dev == nullptr || cell_host == nullptr) return fail_arg("bad arguments");
    if (!(radius > 0.0)) return fail_arg("radius must be positive");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (E == 0) { DYNB_CUDA_OK(cudaMemsetAsync(count_dev, 0, 8, s)); return DYNB_OK; }
    int64_t need;
    dynb_select_workspace_bytes(2 * E, &need);
    if (workspace_dev == nullptr || workspace_bytes < need) return fail_arg("workspace too small (dynb_select_workspace_bytes(2*E))");
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    uint32_t* keep = reinterpret_cast<uint32_t*>(ws);
    uint32_t* excl = keep + (E + 1);
    uint32_t* sums = reinterpret_cast<uint32_t*>(ws + align_up((2 * E + 2) * 4, 256));
    uint32_t* total = reinterpret_cast<uint32_t*>(ws + need - 256);
    Cell9 c;
    for (int i = 0; i < 9; i++) c.c[i] = cell_host[i];
    const float r2 = static_cast<float>(radius * radius);  // dist_graph_ops_kernels.cu:84
    edge_keep_flags_kernel<<<nblk(E), 256, 0, s>>>(edges_dev, edges_dev + E, shifts_f32_dev, pos_dev, c, r2, E, keep);
    DYNB_CUDA_OK((exclusive_scan<uint32_t, uint32_t>(keep, excl, nullptr, E, sums, total, s)));
    u32_total_to_i64_kernel<<<1, 1, 0, s>>>(total, count_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_filter_edges_fill(const int64_t* edges_dev, const void* shifts_raw_dev, int shift_row_bytes, int64_t E,
                                      int64_t E_out, int64_t* edges_out_dev, void* shifts_out_dev, const void* workspace_dev,
                                      void* stream)
{
    if (E < 0 || E_out < 0 || shift_row_bytes <= 0) return fail_arg("bad arguments");
    if (E == 0 || E_out == 0) return DYNB_OK;
    const unsigned char* ws = static_cast<const unsigned char*>(workspace_dev);
    const uint32_t* keep = reinterpret_cast<const uint32_t*>(ws);
    const uint32_t* excl = keep + (E + 1);
    edge_compact_kernel<<<nblk(E), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        edges_dev, static_cast<const unsigned char*>(shifts_raw_dev), shift_row_bytes, keep, excl, E, E_out, edges_out_dev,
        static_cast<unsigned char*>(shifts_out_dev));
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}
