// KD-tree partition for B200 (sm_100a): recursive bisection along the widest axis, all segments of
// a level at once.
//
// Replaces kdtree_bisect_cuda (dynamis_state/src/csrc/partition/kdtree.cpp:9-26,
// kdtree_kernels.cu:28-467; host recursion of the same rule: kdtree_partitioner.cpp:10-50).
// Per level: bounding box of every segment -> widest axis (first axis on ties) -> sort by
// (segment, coordinate) -> split each segment that still has more than one part at
//   equal counts:  mid = clamp(size / 2, 1, size - 1)
//   weights:       first position whose inclusive prefix weight reaches half the segment's weight,
//                  clamped to [1, size - 1]
// -> left / right child segment.  ceil(log2 W) levels, then segment -> label.
// What differs from the reference: the sort is our stable radix sort on (segment << 32 | ordered
// coordinate bits), so atoms with equal coordinates keep ascending index order (the reference's
// at::sort leaves ties unspecified); weights are summed as exact 64-bit integers, where the
// reference converts them to float32 and uses a float cumulative sum (identical while every partial
// sum is below 2^24; beyond that the reference's own result depends on the summation order); bounding
// boxes are reduced per block in shared memory instead of one atomic per atom and axis.
// With equal counts the sort is not needed at all: the cut of a segment is the atom of rank mid in
// (coordinate, index) order, found for all segments of a level at once by the digit-by-digit selection
// of select.cuh on (segment, coordinate, index); an atom goes right when it is not in front of its
// segment's cut.  Weighted cuts keep the sorted path (they need ranks for the clamp).

#include <vector>

#include "common.cuh"
#include "scan.cuh"
#include "select.cuh"

namespace dynb {

constexpr int KD_MAX_SEGS_SMEM = 256;

struct KdSeg {            // per segment of the current level
    int32_t parts;        // ranks this segment still has to be cut into
    int32_t child_left;   // segment ids at the next level
    int32_t child_right;
    int32_t pad;
};

// starts[s] = atoms in segments before s (sorted order puts segments in id order); boxes reset
__global__ void kd_level_init_kernel(int S, const long long* __restrict__ seg_size, long long* __restrict__ seg_start,
                                     uint32_t* __restrict__ box)
{
    if (threadIdx.x == 0) {
        long long acc = 0;
        for (int s = 0; s < S; s++) { seg_start[s] = acc; acc += seg_size[s]; }
        seg_start[S] = acc;
    }
    for (int k = threadIdx.x; k < S * 6; k += blockDim.x) box[k] = ((k % 6) < 3) ? 0xffffffffu : 0u;
}

// box[s*6 + 0..2] = min, +3..5 = max of the ordered-integer images of the coordinates
__global__ void __launch_bounds__(256)
kd_bbox_kernel(const float* __restrict__ pos, const int32_t* __restrict__ seg_id, int64_t n, int S, uint32_t* __restrict__ box)
{
    __shared__ uint32_t sbox[KD_MAX_SEGS_SMEM * 6];
    const bool in_smem = S <= KD_MAX_SEGS_SMEM;
    if (in_smem) {
        for (int k = threadIdx.x; k < S * 6; k += blockDim.x) sbox[k] = ((k % 6) < 3) ? 0xffffffffu : 0u;
        __syncthreads();
    }
    uint32_t* tgt = in_smem ? sbox : box;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int s = seg_id[i];
#pragma unroll
        for (int d = 0; d < 3; d++) {
            const uint32_t o = ordered_u32(pos[3 * i + d]);
            // most atoms of a warp sit in the same segment: skip the atomic when it cannot change anything
            if (o < tgt[s * 6 + d]) atomicMin(&tgt[s * 6 + d], o);
            if (o > tgt[s * 6 + 3 + d]) atomicMax(&tgt[s * 6 + 3 + d], o);
        }
    }
    if (in_smem) {
        __syncthreads();
        for (int k = threadIdx.x; k < S * 6; k += blockDim.x) {
            if ((k % 6) < 3) { if (sbox[k] != 0xffffffffu) atomicMin(&box[k], sbox[k]); }
            else if (sbox[k] != 0u) atomicMax(&box[k], sbox[k]);
        }
    }
}

// widest axis of the segment (kdtree_kernels.cu:58-70: strict '>' keeps the first axis on ties)
__device__ __forceinline__ int kd_axis(const uint32_t* __restrict__ box, int s)
{
    float best = -1.0f;
    int axis = 0;
#pragma unroll
    for (int d = 0; d < 3; d++) {
        const float ext = unordered_f32(box[s * 6 + 3 + d]) - unordered_f32(box[s * 6 + d]);
        if (ext > best) { best = ext; axis = d; }
    }
    return axis;
}

__global__ void __launch_bounds__(256)
kd_keys_kernel(const float* __restrict__ pos, const int32_t* __restrict__ seg_id, int64_t n, const uint32_t* __restrict__ box,
               uint64_t* __restrict__ keys, uint32_t* __restrict__ vals)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int s = seg_id[i];
    const int axis = kd_axis(box, s);
    keys[i] = ((uint64_t)(uint32_t)s << 32) | (uint64_t)ordered_u32(pos[3 * i + axis]);
    vals[i] = (uint32_t)i;
}

__global__ void __launch_bounds__(256)
kd_gather_weights_kernel(const int64_t* __restrict__ w, const uint32_t* __restrict__ vals, int64_t* __restrict__ sorted_w, int64_t n)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) sorted_w[i] = w[vals[i]];
}

// mid[s] and the sizes of the next level's segments.  excl (n + 1 entries, or nullptr for equal counts):
// exclusive prefix of the sorted weights, excl[n] = total.
__global__ void __launch_bounds__(256)
kd_split_kernel(int S, const KdSeg* __restrict__ seg, const long long* __restrict__ seg_size, const long long* __restrict__ seg_start,
                const long long* __restrict__ excl, long long* __restrict__ mid, long long* __restrict__ next_size,
                long long* __restrict__ thresholds /* or nullptr: 1 + atoms in front of the cut, in sorted order */)
{
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= S) return;
    const KdSeg g = seg[s];
    const long long sz = seg_size[s];
    long long m;
    if (g.parts <= 1 || sz <= 1) {
        m = sz;  // kdtree_kernels.cu:110-111, 135-138: everything goes to the left child
    } else if (excl == nullptr) {
        m = min(max(sz / 2, 1ll), sz - 1);
    } else {
        const long long start = seg_start[s];
        const long long base = excl[start];                      // weight in front of the segment
        const long long total = excl[start + sz] - base;
        long long lo = 0, hi = sz - 1;                           // kdtree_kernels.cu:145-153 with exact integers:
        while (lo < hi) {                                        // cumsum < base + total / 2  <=>  2 (cumsum - base) < total
            const long long k = (lo + hi) / 2;
            if (2 * (excl[start + k + 1] - base) < total) lo = k + 1; else hi = k;
        }
        m = min(max(lo, 1ll), sz - 1);
    }
    mid[s] = m;
    if (thresholds != nullptr) thresholds[s] = seg_start[s] + m + 1;
    if (g.child_left == g.child_right) {
        next_size[g.child_left] = sz;
    } else {
        next_size[g.child_left] = m;
        next_size[g.child_right] = sz - m;
    }
}

__global__ void __launch_bounds__(256)
kd_assign_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n, const KdSeg* __restrict__ seg,
                 const long long* __restrict__ seg_start, const long long* __restrict__ mid, int32_t* __restrict__ new_seg_id)
{
    const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n) return;
    const int s = (int)(keys[q] >> 32);
    const KdSeg g = seg[s];
    new_seg_id[vals[q]] = (q - seg_start[s] < mid[s]) ? g.child_left : g.child_right;
}

// equal counts without a sort: an atom goes right when its (coordinate, index) is not in front of its segment's cut
__global__ void __launch_bounds__(256)
kd_assign_select_kernel(const uint64_t* __restrict__ keys, int64_t n, int idx_bits, const SelSplit* __restrict__ cut,
                        const KdSeg* __restrict__ seg, int32_t* __restrict__ new_seg_id)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t key = keys[i];
    const int s = (int)(key >> 32);
    const SelSplit c = cut[s];
    const u128 C = ((u128)key << idx_bits) | (u128)(uint64_t)i;
    const bool right = !c.dead && C >= sel_prefix(c);
    const KdSeg g = seg[s];
    new_seg_id[i] = right ? g.child_right : g.child_left;
}

__global__ void __launch_bounds__(256)
kd_label_kernel(const int32_t* __restrict__ seg_id, const int64_t* __restrict__ base_label, int64_t* __restrict__ labels, int64_t n)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) labels[i] = base_label[seg_id[i]];
}

struct KdLayout { int64_t keys, vals, seg_a, seg_b, sorted_w, excl, sums, tree, size_a, size_b, start, mid, thr, box, base_label, rs, sel_state, sel_hist, total; };
static KdLayout kd_layout(int64_t n, int64_t W)
{
    KdLayout L;
    int64_t o = 0;
    auto take = [&](int64_t b) { int64_t r = o; o = align_up(o + b, 256); return r; };
    int64_t rs_bytes = 0;
    dynb_radix_sort_workspace_bytes(n, &rs_bytes);
    L.keys = take(n * 8);
    L.vals = take(n * 4);
    L.seg_a = take(n * 4);
    L.seg_b = take(n * 4);
    L.sorted_w = take(n * 8);
    L.excl = take((n + 1) * 8);
    L.sums = take((int64_t)(scan_num_tiles(n + 1) + 1) * 8);
    L.tree = take(W * (int64_t)sizeof(KdSeg));
    L.size_a = take((W + 1) * 8);
    L.size_b = take((W + 1) * 8);
    L.start = take((W + 2) * 8);
    L.mid = take((W + 1) * 8);
    L.thr = take((W + 1) * 8);
    L.box = take(W * 6 * 4);
    L.base_label = take((W + 1) * 8);
    L.rs = take(rs_bytes);
    L.sel_state = take(2 * SEL_MAX_SPLITS * (int64_t)sizeof(SelSplit));
    L.sel_hist = take(2 * SEL_HIST_BYTES);
    L.total = o;
    return L;
}

}  // namespace dynb

using namespace dynb;

extern "C" int dynb_kdtree_workspace_bytes(int64_t n_atoms, int64_t W, int64_t* bytes)
{
    if (n_atoms < 0 || W < 1 || bytes == nullptr || n_atoms >= (1ll << 32) - 1 || W > (1ll << 20)) return fail_arg("bad arguments");
    *bytes = kd_layout(std::max<int64_t>(n_atoms, 1), W).total;
    return DYNB_OK;
}

extern "C" int dynb_kdtree_partition(const float* pos_dev, int64_t n_atoms, const int64_t* weights_dev, int64_t W,
                                     int64_t* labels_dev, int method, void* workspace_dev, int64_t workspace_bytes, void* stream)
{
    if (n_atoms < 0) return fail_arg("n_atoms must be non-negative");
    if (method != 0 && method != 1) return fail_arg("method must be 0 (automatic) or 1 (sorted cuts)");
    if (W < 1 || W > (1ll << 20)) return fail_arg("W must be >= 1");
    if (n_atoms == 0) return DYNB_OK;
    if (pos_dev == nullptr || labels_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t n = n_atoms;
    const unsigned nbk = (unsigned)((n + 255) / 256);
    if (W == 1) {  // kdtree_kernels.cu:268-270
        DYNB_CUDA_OK(cudaMemsetAsync(labels_dev, 0, (size_t)n * 8, s));
        return DYNB_OK;
    }
    if (workspace_dev == nullptr) return fail_arg("null workspace");
    const KdLayout L = kd_layout(n, W);
    if (workspace_bytes < L.total) return fail_arg("workspace too small (see dynb_kdtree_workspace_bytes)");
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    uint64_t* keys = reinterpret_cast<uint64_t*>(ws + L.keys);
    uint32_t* vals = reinterpret_cast<uint32_t*>(ws + L.vals);
    int32_t* seg_cur = reinterpret_cast<int32_t*>(ws + L.seg_a);
    int32_t* seg_next = reinterpret_cast<int32_t*>(ws + L.seg_b);
    int64_t* sorted_w = reinterpret_cast<int64_t*>(ws + L.sorted_w);
    long long* excl = reinterpret_cast<long long*>(ws + L.excl);
    long long* sums = reinterpret_cast<long long*>(ws + L.sums);
    KdSeg* tree = reinterpret_cast<KdSeg*>(ws + L.tree);
    long long* size_cur = reinterpret_cast<long long*>(ws + L.size_a);
    long long* size_next = reinterpret_cast<long long*>(ws + L.size_b);
    long long* start = reinterpret_cast<long long*>(ws + L.start);
    long long* mid = reinterpret_cast<long long*>(ws + L.mid);
    long long* thr = reinterpret_cast<long long*>(ws + L.thr);
    const bool by_selection = (weights_dev == nullptr) && W <= SEL_MAX_SPLITS && method == 0;
    uint32_t* box = reinterpret_cast<uint32_t*>(ws + L.box);
    int64_t* base_label = reinterpret_cast<int64_t*>(ws + L.base_label);
    int64_t rs_bytes = 0;
    dynb_radix_sort_workspace_bytes(n, &rs_bytes);

    // the tree of part counts, level by level (kdtree_kernels.cu:215-262)
    int levels = 0;
    for (int64_t v = 1; v < W; v <<= 1) levels++;
    std::vector<int32_t> cur_parts = {(int32_t)W};
    DYNB_CUDA_OK(cudaMemsetAsync(seg_cur, 0, (size_t)n * 4, s));
    const long long n_ll = n;
    DYNB_CUDA_OK(cudaMemcpyAsync(size_cur, &n_ll, 8, cudaMemcpyHostToDevice, s));
    const int grid_stride = (int)std::min<int64_t>(nbk, (int64_t)sm_count_cached() * 8);
    for (int l = 0; l < levels; l++) {
        const int S = (int)cur_parts.size();
        std::vector<KdSeg> segs(S);
        std::vector<int32_t> next_parts;
        for (int k = 0; k < S; k++) {
            segs[k].parts = cur_parts[k];
            segs[k].pad = 0;
            if (cur_parts[k] <= 1) {
                segs[k].child_left = segs[k].child_right = (int32_t)next_parts.size();
                next_parts.push_back(cur_parts[k]);
            } else {
                const int32_t lp = cur_parts[k] / 2;
                segs[k].child_left = (int32_t)next_parts.size();
                next_parts.push_back(lp);
                segs[k].child_right = (int32_t)next_parts.size();
                next_parts.push_back(cur_parts[k] - lp);
            }
        }
        // small pageable source: staged by cudaMemcpyAsync before it returns
        DYNB_CUDA_OK(cudaMemcpyAsync(tree, segs.data(), (size_t)S * sizeof(KdSeg), cudaMemcpyHostToDevice, s));
        kd_level_init_kernel<<<1, 256, 0, s>>>(S, size_cur, start, box);
        kd_bbox_kernel<<<grid_stride, 256, 0, s>>>(pos_dev, seg_cur, n, S, box);
        kd_keys_kernel<<<nbk, 256, 0, s>>>(pos_dev, seg_cur, n, box, keys, vals);
        int seg_bits = 0;
        while ((1 << seg_bits) < S) seg_bits++;
        if (by_selection) {
            kd_split_kernel<<<(S + 255) / 256, 256, 0, s>>>(S, tree, size_cur, start, nullptr, mid, size_next, thr);
            int idx_bits = 0;
            const SelSplit* cut = nullptr;
            int rc = sel_select_splits(keys, 32 + seg_bits, nullptr, n, S, W, thr, ws + L.sel_state, ws + L.sel_hist, &idx_bits, &cut, true, s);
            if (rc) return rc;
            kd_assign_select_kernel<<<nbk, 256, 0, s>>>(keys, n, idx_bits, cut, tree, seg_next);
        } else {
            const int end_bit = std::min(64, ((32 + seg_bits + 7) / 8) * 8);
            int rc = dynb_radix_sort_pairs(keys, vals, n, 0, end_bit, ws + L.rs, rs_bytes, s);
            if (rc) return rc;
            const long long* excl_arg = nullptr;
            if (weights_dev != nullptr) {
                kd_gather_weights_kernel<<<nbk, 256, 0, s>>>(weights_dev, vals, sorted_w, n);
                DYNB_CUDA_OK((exclusive_scan<long long, long long>(reinterpret_cast<long long*>(sorted_w), excl, nullptr, n, sums, excl + n, s)));
                excl_arg = excl;
            }
            kd_split_kernel<<<(S + 255) / 256, 256, 0, s>>>(S, tree, size_cur, start, excl_arg, mid, size_next, nullptr);
            kd_assign_kernel<<<nbk, 256, 0, s>>>(keys, vals, n, tree, start, mid, seg_next);
        }
        std::swap(seg_cur, seg_next);
        std::swap(size_cur, size_next);
        cur_parts.swap(next_parts);
    }
    std::vector<int64_t> base(cur_parts.size());
    int64_t label = 0;
    for (size_t k = 0; k < cur_parts.size(); k++) { base[k] = label; label += cur_parts[k]; }
    DYNB_CUDA_OK(cudaMemcpyAsync(base_label, base.data(), base.size() * 8, cudaMemcpyHostToDevice, s));
    kd_label_kernel<<<nbk, 256, 0, s>>>(seg_cur, base_label, labels_dev, n);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}
