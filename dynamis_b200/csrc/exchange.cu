// Halo exchange kernels for B200 (sm_100a): row pack, fused gather + peer store over NVLink,
// generation signalling with bounded waits, deterministic reverse accumulation.
//
// Replaces, behind the C ABI in dynb.h:
//   push_buffer_create                   dynamis_model/src/csrc/push_buffer.cu:6-105
//   gather_and_push / ghost-grad push    dynamis_model/src/csrc/exchange/ipc_exchange_kernels.cu:40-226
//   record_push_complete / wait_for_pushes  dynamis_model/src/csrc/exchange/ipc_exchanger.cpp:784-828
//   index_add_ of received gradients     dynamis_model/src/csrc/exchanger.cu:111-117
//
// Differences by design: a thread moves 16 bytes (not one float) and finds its peer from a table
// of at most W entries staged in shared memory (not a per-float binary search over int64 offsets);
// peers are signalled with a release store of the generation and awaited by an acquire spin with a
// time budget that ends in a status word (the reference waits without bound); the reverse
// accumulation walks an inverse CSR in fixed peer order (no float atomics, bit-reproducible).
// No load ever reads a peer's memory: peers only receive stores.

#include "common.cuh"
#include "scan.cuh"

#include <string.h>

namespace dynb {

// ------------------------------------------------------------------------------------------ pack
template <typename V>
__global__ void __launch_bounds__(256)
pack_rows_kernel(const V* __restrict__ in, int64_t n_rows_in, int64_t q /* V per row */, const int64_t* __restrict__ locs,
                 int64_t n, V* __restrict__ out, uint32_t* __restrict__ bad)
{
    const int64_t total = n * q;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / q, col = i - row * q;
        const int64_t src = locs[row];
        if (src < 0 || src >= n_rows_in) { if (bad) atomicOr(bad, 1u); continue; }
        out[i] = in[src * q + col];
    }
}

// ------------------------------------------------------------------------------------------ push
constexpr int PUSH_MAX_TARGETS = 128;

struct PushTable {
    const dynb_push_target* targets;  // device array
    int n;
};

// rows [t.start, t.start + t.count) of the logical send list go to peer t at row t.remote_row_offset.
// row_index == nullptr: the logical list is rows src_row_base + i of x (ghost-gradient push);
// otherwise row i of the list is x[row_index[i]] (forward push).  A source row outside [0, n_rows_in) or
// a destination row outside [0, t.remote_rows) is skipped and reported through *bad.
template <typename V>
__global__ void __launch_bounds__(256)
push_rows_kernel(const V* __restrict__ x, int64_t n_rows_in, int64_t q, const int64_t* __restrict__ row_index,
                 int64_t src_row_base, PushTable tab, int64_t total_rows, uint32_t* __restrict__ bad)
{
    __shared__ dynb_push_target st[PUSH_MAX_TARGETS];
    for (int k = threadIdx.x; k < tab.n; k += blockDim.x) st[k] = tab.targets[k];
    __syncthreads();
    const int64_t total = total_rows * q;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / q, col = i - row * q;
        int t = 0;
        while (t < tab.n && !(row >= st[t].start && row < st[t].start + st[t].count)) t++;
        if (t == tab.n) continue;  // rows outside every segment are not sent
        const int64_t src = row_index ? row_index[row] : src_row_base + row;
        const int64_t drow = st[t].remote_row_offset + (row - st[t].start);
        if (src < 0 || src >= n_rows_in || drow < 0 || drow >= st[t].remote_rows) {
            if (bad) atomicOr(bad, 1u);
            continue;
        }
        V* dst = reinterpret_cast<V*>(st[t].remote_ptr);
        dst[drow * q + col] = x[src * q + col];
    }
    __threadfence_system();  // peer stores performed before this kernel's completion is signalled
}

// ------------------------------------------------------------------------------------------ handshake records
// Every rank keeps, inside its exchange allocation, one 16-byte record per (direction, generation
// parity, sender): {generation, announced slot, drift word, pad}.  A sender stores slot and drift,
// fences, then release-stores the generation: whoever acquires the generation also sees the rest and
// every row the sender pushed before.  Two parities because a peer may already be one generation
// ahead (it cannot be two ahead: that needs this rank's next signal).  Records are only ever written
// by stores from the sender and read locally by the owner.
struct FlagRec {
    uint32_t gen, slot, drift, pad;
};

__device__ __forceinline__ FlagRec* local_rec(const dynb_halo_ctx& c, int dir, uint32_t parity, int sender)
{
    return reinterpret_cast<FlagRec*>(static_cast<unsigned char*>(c.local_base) + c.local_flags_off) +
           ((dir * 2 + (int)parity) * c.world_size + sender);
}

__device__ __forceinline__ FlagRec* remote_rec(const dynb_halo_ctx& c, const dynb_halo_peer& p, int dir, uint32_t parity)
{
    return reinterpret_cast<FlagRec*>(static_cast<unsigned char*>(p.remote_base) + p.flags_off) +
           ((dir * 2 + (int)parity) * c.world_size + c.rank);
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Called by every thread of one block: thread k signals rank k (its own record included, so that the
// OR over the records after the wait covers this rank's drift word too).
__device__ void signal_all(const dynb_halo_ctx& c, int dir, uint32_t gen, uint32_t announce)
{
    const uint32_t drift = c.drift_local ? (uint32_t)*reinterpret_cast<const volatile int32_t*>(c.drift_local) : 0u;
    for (int k = threadIdx.x; k < c.world_size; k += blockDim.x) {
        FlagRec* r;
        if (k == c.rank) r = local_rec(c, dir, gen & 1u, k);
        else if (c.peers[k].remote_base != nullptr) r = remote_rec(c, c.peers[k], dir, gen & 1u);
        else continue;
        volatile FlagRec* vr = r;
        vr->slot = announce;
        vr->drift = drift;
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(&r->gen), "r"(gen) : "memory");
    }
}

// Called by every thread of a block.  Thread k waits until rank k's record of this generation has
// arrived (wrap-safe compare) or the budget runs out; on expiry 1 + k is recorded in status word 0
// (device and, when given, mapped host copy) and the wait ends: nothing traps, nothing spins forever.
// Returns true to every thread when all records arrived.
__device__ bool wait_all(const dynb_halo_ctx& c, int dir, uint32_t gen, unsigned long long budget_ns)
{
    int ok = 1;
    for (int k = threadIdx.x; k < c.world_size; k += blockDim.x) {
        if (k == c.rank || c.peers[k].remote_base == nullptr) continue;
        const FlagRec* r = local_rec(c, dir, gen & 1u, k);
        const unsigned long long t0 = globaltimer_ns();
        unsigned long long spins = 0;
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&r->gen) : "memory");
            if ((int32_t)(v - gen) >= 0) break;
            spins++;
            if ((spins & 63) == 0 && (globaltimer_ns() - t0 > budget_ns || spins > (1ull << 34))) {
                atomicCAS(c.status_dev, 0u, (uint32_t)(1 + k));
                if (c.status_host != nullptr) {
                    *reinterpret_cast<volatile uint32_t*>(c.status_host) = (uint32_t)(1 + k);
                    __threadfence_system();
                }
                ok = 0;
                break;
            }
            __nanosleep(64);
        }
    }
    return __syncthreads_and(ok) != 0;
}

// OR of the drift words all ranks attached to this generation (warp 0 of one block, after wait_all).
__device__ void drift_or(const dynb_halo_ctx& c, int dir, uint32_t gen)
{
    if (c.drift_global == nullptr || threadIdx.x >= 32) return;
    uint32_t acc = 0;
    for (int k = threadIdx.x; k < c.world_size; k += 32) {
        if (k != c.rank && c.peers[k].remote_base == nullptr) continue;
        acc |= reinterpret_cast<const volatile FlagRec*>(local_rec(c, dir, gen & 1u, k))->drift;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc |= __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) *c.drift_global = (int32_t)acc;
}

__device__ __forceinline__ void report_bad(const dynb_halo_ctx& c)
{
    atomicOr(c.status_dev + 1, 1u);
    if (c.status_host != nullptr) reinterpret_cast<volatile uint32_t*>(c.status_host)[1] = 1u;
}

// The block that finishes last signals the peers (every block has fenced its peer stores before it
// counts itself in) and leaves the counter at zero for the next launch.
__device__ void last_block_signals(const dynb_halo_ctx& c, int dir, uint32_t gen, uint32_t announce)
{
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(c.done_counter, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (s_last) {
        __threadfence();
        signal_all(c, dir, gen, announce);
        if (threadIdx.x == 0) *c.done_counter = 0u;
    }
}

// byte range [0, bytes) copied by `parts` blocks, this block being `part`; vb = 16, 4 or 1 is the
// widest unit both pointers are aligned to.  Blocks interleave (block-sized pieces, grid stride): all
// resident blocks then stream through neighbouring addresses, which HBM serves about a quarter faster
// than one far-apart chunk per block.
__device__ void copy_span(unsigned char* __restrict__ dst, const unsigned char* __restrict__ src, int64_t bytes, int vb,
                          int64_t part, int64_t parts)
{
    if (vb == 16) {
        constexpr int U = 8;
        const int64_t n = bytes >> 4;
        const uint4* s = reinterpret_cast<const uint4*>(src);
        uint4* d = reinterpret_cast<uint4*>(dst);
        const int64_t bd = blockDim.x, step = parts * bd * U;
        int64_t i = part * bd * U + threadIdx.x;
        for (; i + (U - 1) * bd < n; i += step) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++) v[u] = __ldcs(s + i + u * bd);
#pragma unroll
            for (int u = 0; u < U; u++) d[i + u * bd] = v[u];
        }
        for (int u = 0; u < U; u++)
            if (i + u * bd < n) d[i + u * bd] = __ldcs(s + i + u * bd);
        if (part == 0) for (int64_t t = (n << 4) + threadIdx.x; t < bytes; t += bd) dst[t] = src[t];
    } else if (vb == 4) {
        const int64_t n = bytes >> 2;
        const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
        uint32_t* d = reinterpret_cast<uint32_t*>(dst);
        for (int64_t i = part * blockDim.x + threadIdx.x; i < n; i += parts * blockDim.x) d[i] = s[i];
        if (part == 0) for (int64_t t = (n << 2) + threadIdx.x; t < bytes; t += blockDim.x) dst[t] = src[t];
    } else {
        for (int64_t i = part * blockDim.x + threadIdx.x; i < bytes; i += parts * blockDim.x) dst[i] = src[i];
    }
}

// Rows of q 16-byte units whose flag is zero, copied one warp per row, R rows in flight per warp.
__device__ void copy_rows_unflagged(uint4* __restrict__ dst, const uint4* __restrict__ src, const uint8_t* __restrict__ flag,
                                    int64_t rows, int64_t q, int64_t part, int64_t parts)
{
    constexpr int R = 4;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int64_t nw = parts * wpb, w = part * wpb + (threadIdx.x >> 5);
    const int64_t lo = rows * w / nw, hi = rows * (w + 1) / nw;
    for (int64_t r0 = lo; r0 < hi; r0 += R) {
        bool ok[R];
#pragma unroll
        for (int k = 0; k < R; k++) ok[k] = (r0 + k < hi) && flag[r0 + k] == 0;
        for (int64_t c = lane; c < q; c += 32) {
            uint4 v[R];
#pragma unroll
            for (int k = 0; k < R; k++)
                if (ok[k]) v[k] = __ldcs(src + (r0 + k) * q + c);
#pragma unroll
            for (int k = 0; k < R; k++)
                if (ok[k]) dst[(r0 + k) * q + c] = v[k];
        }
    }
}

struct PeerSeg {
    unsigned char* dst;   // where row `start` of the segment lands at the peer
    int64_t start, end;   // rows [start, end) of the logical list
};

__device__ __forceinline__ int find_seg(const PeerSeg* seg, int n, int64_t row)
{
    int t = 0;
    while (t < n && !(row >= seg[t].start && row < seg[t].end)) t++;
    return t;
}

// Units [0, total) (V-wide pieces of the logical push list's rows) stored into the peers by `parts` blocks,
// this block being `part`, interleaved like copy_span.  INDEXED: logical row i is x[index[i]] (forward),
// else x[src_row_base + i] (ghost-gradient rows).
// `stride` > 0: the block-sized pieces are visited in the order (k * stride) mod pieces (stride coprime to the
// number of pieces, about 0.62 of it), so that at any moment the pieces in flight are spread over the whole
// list — over all peers — instead of all ranks storing into the same peer's segment at the same time.
template <typename V, bool INDEXED>
__device__ void push_units(const dynb_halo_ctx& c, const V* __restrict__ x, int64_t n_rows_in, int64_t q,
                           const int64_t* __restrict__ index, int64_t src_row_base, const PeerSeg* seg, int nseg,
                           int64_t total, int64_t part, int64_t parts, unsigned long long stride)
{
    constexpr int U = 4;
    const int64_t bd = blockDim.x, piece = bd * U;
    const unsigned long long pieces = (unsigned long long)((total + piece - 1) / piece);
    const bool small = total < (1ll << 32);
    for (unsigned long long k = (unsigned long long)part; k < pieces; k += (unsigned long long)parts) {
        const int64_t base = (int64_t)(stride ? (k * stride) % pieces : k) * piece + threadIdx.x;
        V v[U];
        V* d[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t i = base + u * bd;
            d[u] = nullptr;
            if (i >= total) continue;
            int64_t row, col;
            if (small) { const uint32_t r32 = (uint32_t)i / (uint32_t)q; row = r32; col = (uint32_t)i - r32 * (uint32_t)q; }
            else { row = i / q; col = i - row * q; }
            const int t = find_seg(seg, nseg, row);
            if (t == nseg) continue;
            const int64_t src = INDEXED ? index[row] : src_row_base + row;
            if (src < 0 || src >= n_rows_in) { report_bad(c); continue; }
            v[u] = x[src * q + col];
            d[u] = reinterpret_cast<V*>(seg[t].dst) + (row - seg[t].start) * q + col;
        }
#pragma unroll
        for (int u = 0; u < U; u++)
            if (d[u] != nullptr) *d[u] = v[u];
    }
}

// stride for push_units: an odd number near 0.618 * pieces that shares no factor with it (0 for short lists)
__device__ unsigned long long scatter_stride(int64_t total, int64_t piece)
{
    const unsigned long long pieces = (unsigned long long)((total + piece - 1) / piece);
    if (pieces < 64) return 0ull;
    unsigned long long s = (unsigned long long)((double)pieces * 0.6180339887) | 1ull;
    for (;;) {
        unsigned long long a = s, b = pieces;
        while (b) { const unsigned long long t = a % b; a = b; b = t; }
        if (a == 1ull) return s;
        s += 2ull;
    }
}

// Forward halo push, first half: rows of the send list -> every peer's ghost region (the result slot the
// peer announced with its previous signal, or its staging buffer), this rank's own rows -> head of the
// result, then the signal.  Even blocks push first and copy second, odd blocks the other way round, so
// that NVLink stores and the HBM copy run side by side.
template <typename V>
__global__ void __launch_bounds__(256, 3)
halo_forward_begin_kernel(dynb_halo_ctx c, const V* __restrict__ x, int64_t n_local, int64_t q, int64_t row_bytes,
                          const int64_t* __restrict__ send_local, int64_t total_send, unsigned char* __restrict__ out_head,
                          int head_vb, uint32_t gen, uint32_t announce, int skip_push)
{
    __shared__ PeerSeg seg[PUSH_MAX_TARGETS];
    for (int k = threadIdx.x; k < c.world_size; k += blockDim.x) {
        const dynb_halo_peer p = c.peers[k];
        PeerSeg s{nullptr, 0, 0};
        if (k != c.rank && p.remote_base != nullptr && p.send_count > 0) {
            // the slot this peer announced for this generation travelled with its previous signal
            const uint32_t slot = reinterpret_cast<const volatile FlagRec*>(local_rec(c, 0, (gen - 1u) & 1u, k))->slot;
            const int64_t tail = slot == 0u ? p.fwd_stage_off[gen & 1u] : p.fwd_ring_tail + (int64_t)(slot - 1u) * p.fwd_ring_stride;
            s.dst = static_cast<unsigned char*>(p.remote_base) + tail + p.fwd_row_offset * row_bytes;
            s.start = p.send_start;
            s.end = p.send_start + p.send_count;
        }
        seg[k] = s;
    }
    __syncthreads();
    const int64_t G = gridDim.x, b = blockIdx.x;
    const int64_t P = (skip_push & 1) ? 0 : total_send * q;
    const unsigned long long stride = (skip_push & 2) ? 0ull : scatter_stride(P, (int64_t)blockDim.x * 4);
    const unsigned char* xs = reinterpret_cast<const unsigned char*>(x);
    const int64_t head_bytes = n_local * row_bytes;
    // Even blocks push first and copy second, odd blocks the other way round: measured on four GPUs (2 M rows
    // of 512 bytes copied, 395 k pushed) 0.52 ms against 0.51 ms for the push alone and 0.37 ms for the copy
    // alone; alternating the two inside every warp gave 0.58 ms, blocks with a fixed role 0.54-0.87 ms.
    if (b & 1) {
        if (out_head != nullptr) copy_span(out_head, xs, head_bytes, head_vb, b, G);
        push_units<V, true>(c, x, n_local, q, send_local, 0, seg, c.world_size, P, b, G, stride);
    } else {
        push_units<V, true>(c, x, n_local, q, send_local, 0, seg, c.world_size, P, b, G, stride);
        if (out_head != nullptr) copy_span(out_head, xs, head_bytes, head_vb, b, G);
    }
    last_block_signals(c, 0, gen, announce);
}

// Forward, second half: bounded wait for every peer's signal of this generation, OR of the drift words,
// and — when the rows arrived in the staging buffer rather than in the result itself — their copy into
// the result's tail.
__global__ void __launch_bounds__(256)
halo_forward_end_kernel(dynb_halo_ctx c, uint32_t gen, unsigned long long budget_ns, const unsigned char* __restrict__ stage,
                        unsigned char* __restrict__ out_tail, int64_t tail_bytes, int tail_vb)
{
    wait_all(c, 0, gen, budget_ns);
    if (blockIdx.x == 0) drift_or(c, 0, gen);
    if (out_tail != nullptr && tail_bytes > 0) copy_span(out_tail, stage, tail_bytes, tail_vb, blockIdx.x, gridDim.x);
}

// Reverse halo, first half: the gradient rows of the ghost atoms -> their owners' receive buffers; the
// gradient rows of owned atoms that receive nothing -> result (has_recv == nullptr: all owned rows); signal.
template <typename V>
__global__ void __launch_bounds__(256, 3)
halo_backward_begin_kernel(dynb_halo_ctx c, const V* __restrict__ g, int64_t n_local, int64_t n_ghost, int64_t q,
                           int64_t row_bytes, const uint8_t* __restrict__ has_recv, unsigned char* __restrict__ out, int out_vb,
                           uint32_t gen)
{
    __shared__ PeerSeg seg[PUSH_MAX_TARGETS];
    for (int k = threadIdx.x; k < c.world_size; k += blockDim.x) {
        const dynb_halo_peer p = c.peers[k];
        PeerSeg s{nullptr, 0, 0};
        if (k != c.rank && p.remote_base != nullptr && p.recv_count > 0) {
            s.dst = static_cast<unsigned char*>(p.remote_base) + p.bwd_off[gen & 1u] + p.bwd_row_offset * row_bytes;
            s.start = p.recv_start;
            s.end = p.recv_start + p.recv_count;
        }
        seg[k] = s;
    }
    __syncthreads();
    const int64_t G = gridDim.x, b = blockIdx.x;
    const int64_t P = n_ghost * q;
    const unsigned long long stride = scatter_stride(P, (int64_t)blockDim.x * 4);
    const unsigned char* gs = reinterpret_cast<const unsigned char*>(g);
    const int64_t own_bytes = n_local * row_bytes;
    // has_recv comes only with 16-byte aligned rows of at least 64 bytes (host side): rows that the second half
    // rewrites anyway are left out of the copy
    if (b & 1) {
        if (has_recv == nullptr) copy_span(out, gs, own_bytes, out_vb, b, G);
        else copy_rows_unflagged(reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(g), has_recv, n_local, row_bytes >> 4, b, G);
        push_units<V, false>(c, g, n_local + n_ghost, q, nullptr, n_local, seg, c.world_size, P, b, G, stride);
    } else {
        push_units<V, false>(c, g, n_local + n_ghost, q, nullptr, n_local, seg, c.world_size, P, b, G, stride);
        if (has_recv == nullptr) copy_span(out, gs, own_bytes, out_vb, b, G);
        else copy_rows_unflagged(reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(g), has_recv, n_local, row_bytes >> 4, b, G);
    }
    last_block_signals(c, 1, gen, 0u);
}

// Reverse, second half: bounded wait, drift OR, then for every owned row named by the send list
// out[row] = g[row] + the received rows that name it, in the fixed order of inv_entries.
template <typename T, typename V, int VW>
__global__ void __launch_bounds__(256, 4)
halo_backward_end_kernel(dynb_halo_ctx c, uint32_t gen, unsigned long long budget_ns, const V* __restrict__ g,
                         const int64_t* __restrict__ rows, const uint32_t* __restrict__ row_first, int64_t n_rows, int64_t q,
                         const V* __restrict__ recv, const int64_t* __restrict__ inv_offsets,
                         const uint32_t* __restrict__ inv_entries, V* __restrict__ out)
{
    // one warp per listed row, R rows in flight; lanes walk the row's V-wide columns.  What does not depend on
    // the peers — the rows' ids and their places in the inverse CSR — is requested before the wait for the warp's
    // first step, so that behind the wait the gradient rows and the received rows are one round of independent loads.
    constexpr int R = 4;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int64_t nw = (int64_t)gridDim.x * wpb, w = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5);
    struct Step { int64_t row[R]; uint32_t b[R], e[R], first[R]; };   // list places fit 32 bits (dynb_inverse_csr)
    auto request = [&](int64_t r0, Step& s) {
#pragma unroll
        for (int k = 0; k < R; k++) {
            s.row[k] = -1;
            s.first[k] = 0;
            if (r0 + k < n_rows) {
                s.row[k] = rows[r0 + k];
                if (row_first != nullptr) s.first[k] = row_first[r0 + k];
            }
        }
#pragma unroll
        for (int k = 0; k < R; k++) {
            s.b[k] = s.e[k] = 0;
            if (s.row[k] >= 0) {
                s.b[k] = (uint32_t)inv_offsets[s.row[k]];
                s.e[k] = (uint32_t)inv_offsets[s.row[k] + 1];
            }
        }
    };
    Step cur;
    int64_t r0 = w * R;
    if (r0 < n_rows) request(r0, cur);
    wait_all(c, 1, gen, budget_ns);
    if (blockIdx.x == 0) drift_or(c, 1, gen);
    while (r0 < n_rows) {
        for (int64_t col = lane; col < q; col += 32) {
            V v[R], f[R];
            bool hf[R];
#pragma unroll
            for (int k = 0; k < R; k++) {
                hf[k] = false;
                if (cur.row[k] >= 0) {
                    v[k] = g[cur.row[k] * q + col];
                    hf[k] = cur.b[k] < cur.e[k];
                    if (hf[k]) f[k] = recv[(int64_t)(row_first != nullptr ? cur.first[k] : inv_entries[cur.b[k]]) * q + col];
                }
            }
#pragma unroll
            for (int k = 0; k < R; k++) {
                if (cur.row[k] < 0) continue;
                T* a = reinterpret_cast<T*>(&v[k]);
                if (hf[k]) {
                    const T* fr = reinterpret_cast<const T*>(&f[k]);
#pragma unroll
                    for (int cc = 0; cc < VW; cc++) a[cc] += fr[cc];
                }
                for (uint32_t j = cur.b[k] + 1; j < cur.e[k]; j++) {
                    const V xx = recv[(int64_t)inv_entries[j] * q + col];
                    const T* xr = reinterpret_cast<const T*>(&xx);
#pragma unroll
                    for (int cc = 0; cc < VW; cc++) a[cc] += xr[cc];
                }
                out[cur.row[k] * q + col] = v[k];
            }
        }
        r0 += nw * R;
        if (r0 < n_rows) request(r0, cur);
    }
}

// A bare handshake (no rows): signal, or wait + drift OR, for one direction.
__global__ void halo_signal_kernel(dynb_halo_ctx c, int dir, uint32_t gen, uint32_t announce)
{
    signal_all(c, dir, gen, announce);
}

__global__ void halo_wait_kernel(dynb_halo_ctx c, int dir, uint32_t gen, unsigned long long budget_ns)
{
    wait_all(c, dir, gen, budget_ns);
    drift_or(c, dir, gen);
}

// ------------------------------------------------------------------------------------------ reverse accumulation
// out[row] = grad[row] + sum over the row's received gradient rows, in the order of inv_entries.
template <typename T, typename V, int VW>
__global__ void __launch_bounds__(256)
unpack_add_rows_kernel(const V* __restrict__ grad, int64_t n_local, int64_t q, const V* __restrict__ recv,
                       const int64_t* __restrict__ inv_offsets, const uint32_t* __restrict__ inv_entries, V* __restrict__ out)
{
    const int64_t total = n_local * q;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / q, col = i - row * q;
        V v = grad[i];
        const int64_t b = inv_offsets[row], e = inv_offsets[row + 1];
        T* a = reinterpret_cast<T*>(&v);
        for (int64_t k = b; k < e; k++) {
            const V r = recv[(int64_t)inv_entries[k] * q + col];
            const T* rr = reinterpret_cast<const T*>(&r);
#pragma unroll
            for (int c = 0; c < VW; c++) a[c] += rr[c];
        }
        out[i] = v;
    }
}

__global__ void __launch_bounds__(256)
inv_keys_kernel(const int64_t* __restrict__ send_local, int64_t total_send, int64_t n_local, uint64_t* __restrict__ keys,
                uint32_t* __restrict__ vals, uint32_t* __restrict__ counts, uint32_t* __restrict__ bad)
{
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= total_send) return;
    int64_t r = send_local[j];
    if (r < 0 || r >= n_local) { atomicOr(bad, 1u); r = 0; }
    else atomicAdd(&counts[r], 1u);
    keys[j] = (uint64_t)r;
    vals[j] = (uint32_t)j;
}

static inline unsigned grid_for(int64_t work, int threads = 256)
{
    const int64_t blocks = (work + threads - 1) / threads;
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>(blocks, (int64_t)sm_count_cached() * 16));
}

// chooses the widest vector that divides the row and matches the pointers' alignment
static inline int vec_bytes(int64_t row_bytes, const void* a, const void* b)
{
    const uintptr_t pa = reinterpret_cast<uintptr_t>(a), pb = reinterpret_cast<uintptr_t>(b);
    if (row_bytes % 16 == 0 && pa % 16 == 0 && pb % 16 == 0) return 16;
    if (row_bytes % 4 == 0 && pa % 4 == 0 && pb % 4 == 0) return 4;
    return 1;
}

}  // namespace dynb

using namespace dynb;

extern "C" int dynb_pack_rows(const void* input_dev, int64_t n_rows_in, int64_t row_bytes, const int64_t* locs_dev, int64_t n,
                              void* out_dev, uint32_t* bad_dev, void* stream)
{
    if (n < 0 || row_bytes <= 0 || n_rows_in < 0) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    if (input_dev == nullptr || locs_dev == nullptr || out_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vb = vec_bytes(row_bytes, input_dev, out_dev);
    const int64_t q = row_bytes / vb;
    const unsigned g = grid_for(n * q);
    if (vb == 16) pack_rows_kernel<uint4><<<g, 256, 0, s>>>(static_cast<const uint4*>(input_dev), n_rows_in, q, locs_dev, n, static_cast<uint4*>(out_dev), bad_dev);
    else if (vb == 4) pack_rows_kernel<uint32_t><<<g, 256, 0, s>>>(static_cast<const uint32_t*>(input_dev), n_rows_in, q, locs_dev, n, static_cast<uint32_t*>(out_dev), bad_dev);
    else pack_rows_kernel<uint8_t><<<g, 256, 0, s>>>(static_cast<const uint8_t*>(input_dev), n_rows_in, q, locs_dev, n, static_cast<uint8_t*>(out_dev), bad_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_push_rows(const void* x_dev, int64_t n_rows_in, int64_t row_bytes, const int64_t* row_index_dev,
                              int64_t src_row_base, const dynb_push_target* targets_dev, int n_targets, int64_t total_rows,
                              int remote_align, uint32_t* bad_dev, void* stream)
{
    if (row_bytes <= 0 || n_targets < 0 || n_targets > PUSH_MAX_TARGETS || total_rows < 0 || n_rows_in < 0) return fail_arg("bad arguments");
    if (total_rows == 0 || n_targets == 0) return DYNB_OK;
    if (x_dev == nullptr || targets_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int vb = vec_bytes(row_bytes, x_dev, x_dev);
    if (remote_align < vb) vb = (remote_align >= 4 && row_bytes % 4 == 0) ? 4 : 1;
    const int64_t q = row_bytes / vb;
    PushTable tab{targets_dev, n_targets};
    const unsigned g = grid_for(total_rows * q);
    if (vb == 16) push_rows_kernel<uint4><<<g, 256, 0, s>>>(static_cast<const uint4*>(x_dev), n_rows_in, q, row_index_dev, src_row_base, tab, total_rows, bad_dev);
    else if (vb == 4) push_rows_kernel<uint32_t><<<g, 256, 0, s>>>(static_cast<const uint32_t*>(x_dev), n_rows_in, q, row_index_dev, src_row_base, tab, total_rows, bad_dev);
    else push_rows_kernel<uint8_t><<<g, 256, 0, s>>>(static_cast<const uint8_t*>(x_dev), n_rows_in, q, row_index_dev, src_row_base, tab, total_rows, bad_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

// ------------------------------------------------------------------------------------------ fused halo exchange
static int check_ctx(const dynb_halo_ctx* c)
{
    if (c == nullptr) return fail_arg("null context");
    if (c->world_size < 1 || c->world_size > PUSH_MAX_TARGETS || c->rank < 0 || c->rank >= c->world_size)
        return fail_arg("world size must be 1..128 and rank inside it");
    if (c->peers == nullptr || c->local_base == nullptr || c->done_counter == nullptr || c->status_dev == nullptr)
        return fail_arg("incomplete context");
    return DYNB_OK;
}

static inline int span_vb(const void* a, const void* b, int64_t)
{
    const uintptr_t u = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
    return (u % 16 == 0) ? 16 : (u % 4 == 0) ? 4 : 1;
}

static inline unsigned fused_grid(int64_t units16)
{
    const int64_t blocks = (units16 + 256 * 8 - 1) / (256 * 8);
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>(blocks, (int64_t)sm_count_cached() * 6));  // two waves of 3 CTAs per SM
}

extern "C" int dynb_halo_forward_begin(const dynb_halo_ctx* ctx, const void* x_dev, int64_t n_local, int64_t row_bytes,
                                       const int64_t* send_local_dev, int64_t total_send, void* out_head_dev, uint32_t gen,
                                       uint32_t announce_slot, int skip_push, void* stream)
{
    if (int rc = check_ctx(ctx)) return rc;
    if (n_local < 0 || row_bytes <= 0 || total_send < 0) return fail_arg("bad arguments");
    if ((n_local > 0 && x_dev == nullptr) || (total_send > 0 && send_local_dev == nullptr)) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vb = vec_bytes(row_bytes, x_dev, x_dev);
    const int64_t q = row_bytes / vb;
    const int hv = span_vb(x_dev, out_head_dev, 0);
    const unsigned g = fused_grid((total_send + (out_head_dev ? n_local : 0)) * row_bytes / 16 + 1);
    unsigned char* oh = static_cast<unsigned char*>(out_head_dev);
    if (vb == 16) halo_forward_begin_kernel<uint4><<<g, 256, 0, s>>>(*ctx, static_cast<const uint4*>(x_dev), n_local, q, row_bytes, send_local_dev, total_send, oh, hv, gen, announce_slot, skip_push);
    else if (vb == 4) halo_forward_begin_kernel<uint32_t><<<g, 256, 0, s>>>(*ctx, static_cast<const uint32_t*>(x_dev), n_local, q, row_bytes, send_local_dev, total_send, oh, hv, gen, announce_slot, skip_push);
    else halo_forward_begin_kernel<uint8_t><<<g, 256, 0, s>>>(*ctx, static_cast<const uint8_t*>(x_dev), n_local, q, row_bytes, send_local_dev, total_send, oh, hv, gen, announce_slot, skip_push);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_halo_forward_end(const dynb_halo_ctx* ctx, uint32_t gen, int64_t timeout_ns, const void* stage_dev,
                                     void* out_tail_dev, int64_t tail_bytes, void* stream)
{
    if (int rc = check_ctx(ctx)) return rc;
    if (timeout_ns <= 0 || tail_bytes < 0) return fail_arg("bad arguments");
    if (out_tail_dev != nullptr && tail_bytes > 0 && stage_dev == nullptr) return fail_arg("null pointer");
    const bool copy = out_tail_dev != nullptr && tail_bytes > 0;
    const unsigned g = copy ? fused_grid(tail_bytes / 16 + 1) : 1u;
    halo_forward_end_kernel<<<g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        *ctx, gen, (unsigned long long)timeout_ns, static_cast<const unsigned char*>(stage_dev),
        static_cast<unsigned char*>(out_tail_dev), tail_bytes, span_vb(stage_dev, out_tail_dev, 0));
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_halo_backward_begin(const dynb_halo_ctx* ctx, const void* grad_dev, int64_t n_local, int64_t n_ghost,
                                        int64_t row_bytes, const uint8_t* has_recv_dev, void* out_dev, uint32_t gen, void* stream)
{
    if (int rc = check_ctx(ctx)) return rc;
    if (n_local < 0 || n_ghost < 0 || row_bytes <= 0) return fail_arg("bad arguments");
    if ((n_local + n_ghost > 0 && grad_dev == nullptr) || (n_local > 0 && out_dev == nullptr)) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vb = vec_bytes(row_bytes, grad_dev, grad_dev);
    const int64_t q = row_bytes / vb;
    const int ov = span_vb(grad_dev, out_dev, 0);
    const uint8_t* hr = (vb == 16 && ov == 16 && row_bytes >= 64) ? has_recv_dev : nullptr;  // short rows: plain copy
    const unsigned g = fused_grid((n_local + n_ghost) * row_bytes / 16 + 1);
    unsigned char* o = static_cast<unsigned char*>(out_dev);
    if (vb == 16) halo_backward_begin_kernel<uint4><<<g, 256, 0, s>>>(*ctx, static_cast<const uint4*>(grad_dev), n_local, n_ghost, q, row_bytes, hr, o, ov, gen);
    else if (vb == 4) halo_backward_begin_kernel<uint32_t><<<g, 256, 0, s>>>(*ctx, static_cast<const uint32_t*>(grad_dev), n_local, n_ghost, q, row_bytes, hr, o, ov, gen);
    else halo_backward_begin_kernel<uint8_t><<<g, 256, 0, s>>>(*ctx, static_cast<const uint8_t*>(grad_dev), n_local, n_ghost, q, row_bytes, hr, o, ov, gen);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_halo_backward_end(const dynb_halo_ctx* ctx, uint32_t gen, int64_t timeout_ns, const void* grad_dev,
                                      const int64_t* rows_dev, const uint32_t* row_first_dev, int64_t n_rows, int64_t feature_dim,
                                      int dtype, const void* recv_dev, const int64_t* inv_offsets_dev,
                                      const uint32_t* inv_entries_dev, void* out_dev, void* stream)
{
    if (int rc = check_ctx(ctx)) return rc;
    if (n_rows < 0 || feature_dim <= 0 || timeout_ns <= 0) return fail_arg("bad arguments");
    if (dtype != DYNB_F32 && dtype != DYNB_F64) return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
    if (n_rows > 0 && (rows_dev == nullptr || out_dev == nullptr || grad_dev == nullptr || inv_offsets_dev == nullptr ||
                       inv_entries_dev == nullptr || recv_dev == nullptr))
        return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned long long bud = (unsigned long long)timeout_ns;
    const int64_t row_bytes = feature_dim * (dtype == DYNB_F64 ? 8 : 4);
    const bool al = (reinterpret_cast<uintptr_t>(out_dev) | reinterpret_cast<uintptr_t>(recv_dev) |
                     reinterpret_cast<uintptr_t>(grad_dev)) % 16 == 0;
    if (dtype == DYNB_F32) {
        if (al && row_bytes % 16 == 0) {
            const int64_t q = row_bytes / 16;
            halo_backward_end_kernel<float, float4, 4><<<grid_for(n_rows * 32), 256, 0, s>>>(
                *ctx, gen, bud, static_cast<const float4*>(grad_dev), rows_dev, row_first_dev, n_rows, q, static_cast<const float4*>(recv_dev),
                inv_offsets_dev, inv_entries_dev, static_cast<float4*>(out_dev));
        } else {
            halo_backward_end_kernel<float, float, 1><<<grid_for(n_rows * 32), 256, 0, s>>>(
                *ctx, gen, bud, static_cast<const float*>(grad_dev), rows_dev, row_first_dev, n_rows, feature_dim, static_cast<const float*>(recv_dev),
                inv_offsets_dev, inv_entries_dev, static_cast<float*>(out_dev));
        }
    } else {
        if (al && row_bytes % 16 == 0) {
            const int64_t q = row_bytes / 16;
            halo_backward_end_kernel<double, double2, 2><<<grid_for(n_rows * 32), 256, 0, s>>>(
                *ctx, gen, bud, static_cast<const double2*>(grad_dev), rows_dev, row_first_dev, n_rows, q, static_cast<const double2*>(recv_dev),
                inv_offsets_dev, inv_entries_dev, static_cast<double2*>(out_dev));
        } else {
            halo_backward_end_kernel<double, double, 1><<<grid_for(n_rows * 32), 256, 0, s>>>(
                *ctx, gen, bud, static_cast<const double*>(grad_dev), rows_dev, row_first_dev, n_rows, feature_dim, static_cast<const double*>(recv_dev),
                inv_offsets_dev, inv_entries_dev, static_cast<double*>(out_dev));
        }
    }
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_halo_signal(const dynb_halo_ctx* ctx, int direction, uint32_t gen, uint32_t announce_slot, void* stream)
{
    if (int rc = check_ctx(ctx)) return rc;
    if (direction < 0 || direction > 2) return fail_arg("direction must be 0, 1 or 2");
    halo_signal_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(*ctx, direction, gen, announce_slot);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_halo_wait(const dynb_halo_ctx* ctx, int direction, uint32_t gen, int64_t timeout_ns, void* stream)
{
    if (int rc = check_ctx(ctx)) return rc;
    if (direction < 0 || direction > 2 || timeout_ns <= 0) return fail_arg("bad arguments");
    halo_wait_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(*ctx, direction, gen, (unsigned long long)timeout_ns);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_host_alloc_mapped(int64_t bytes, void** host_ptr_out, void** dev_ptr_out)
{
    if (bytes <= 0 || host_ptr_out == nullptr || dev_ptr_out == nullptr) return fail_arg("bad arguments");
    void* h = nullptr;
    DYNB_CUDA_OK(cudaHostAlloc(&h, (size_t)bytes, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(h, 0, (size_t)bytes);
    void* d = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&d, h, 0);
    if (e != cudaSuccess) { cudaFreeHost(h); return fail_cuda(e, "cudaHostGetDevicePointer"); }
    *host_ptr_out = h;
    *dev_ptr_out = d;
    return DYNB_OK;
}

extern "C" int dynb_host_free_mapped(void* host_ptr)
{
    if (host_ptr == nullptr) return DYNB_OK;
    DYNB_CUDA_OK(cudaFreeHost(host_ptr));
    return DYNB_OK;
}

extern "C" int dynb_inverse_csr_workspace_bytes(int64_t total_send, int64_t n_local, int64_t* bytes)
{
    if (total_send < 0 || n_local < 0 || bytes == nullptr) return fail_arg("bad arguments");
    int64_t rs = 0;
    dynb_radix_sort_workspace_bytes(std::max<int64_t>(total_send, 1), &rs);
    *bytes = align_up(std::max<int64_t>(total_send, 1) * 8, 256) + align_up((n_local + 2) * 4, 256) +
             align_up((int64_t)(scan_num_tiles(n_local + 2) + 1) * 8, 256) + rs + 256;
    return DYNB_OK;
}

// inv_offsets_dev [n_local+1] int64, inv_entries_dev [total_send] uint32: the positions j of the
// send list that name local row i, ascending in j (= ascending peer), for every row i.
extern "C" int dynb_inverse_csr(const int64_t* send_local_dev, int64_t total_send, int64_t n_local, int64_t* inv_offsets_dev,
                                uint32_t* inv_entries_dev, uint32_t* bad_dev, void* workspace_dev, int64_t workspace_bytes,
                                void* stream)
{
    if (total_send < 0 || n_local < 0 || inv_offsets_dev == nullptr || bad_dev == nullptr) return fail_arg("bad arguments");
    if (n_local >= (1ll << 32) || total_send >= (1ll << 32)) return fail_arg("sizes must stay below 2^32");
    int64_t need;
    dynb_inverse_csr_workspace_bytes(total_send, n_local, &need);
    if (workspace_dev == nullptr || workspace_bytes < need) return fail_arg("workspace too small (see dynb_inverse_csr_workspace_bytes)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    int64_t o = 0;
    uint64_t* keys = reinterpret_cast<uint64_t*>(ws + o); o += align_up(std::max<int64_t>(total_send, 1) * 8, 256);
    uint32_t* counts = reinterpret_cast<uint32_t*>(ws + o); o += align_up((n_local + 2) * 4, 256);
    long long* sums = reinterpret_cast<long long*>(ws + o); o += align_up((int64_t)(scan_num_tiles(n_local + 2) + 1) * 8, 256);
    unsigned char* rs = ws + o;
    DYNB_CUDA_OK(cudaMemsetAsync(counts, 0, (size_t)(n_local + 2) * 4, s));
    DYNB_CUDA_OK(cudaMemsetAsync(bad_dev, 0, 4, s));
    if (total_send > 0) {
        inv_keys_kernel<<<(unsigned)((total_send + 255) / 256), 256, 0, s>>>(send_local_dev, total_send, n_local, keys,
                                                                           inv_entries_dev, counts, bad_dev);
        int bits = 8;
        while (bits < 64 && (1ull << bits) < (uint64_t)std::max<int64_t>(n_local, 1)) bits += 8;
        int rc = dynb_radix_sort_pairs(keys, inv_entries_dev, total_send, 0, bits, rs, need - o, stream);
        if (rc) return rc;
    }
    DYNB_CUDA_OK((exclusive_scan<uint32_t, long long>(counts, reinterpret_cast<long long*>(inv_offsets_dev), nullptr, n_local + 1,
                                                       sums, nullptr, s)));
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_unpack_add_rows(const void* grad_dev, int64_t n_local, int64_t feature_dim, int dtype, const void* recv_dev,
                                    const int64_t* inv_offsets_dev, const uint32_t* inv_entries_dev, void* out_dev, void* stream)
{
    if (n_local < 0 || feature_dim <= 0) return fail_arg("bad arguments");
    if (dtype != DYNB_F32 && dtype != DYNB_F64) return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
    if (n_local == 0) return DYNB_OK;
    if (grad_dev == nullptr || out_dev == nullptr || inv_offsets_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t row_bytes = feature_dim * (dtype == DYNB_F64 ? 8 : 4);
    const bool al = (reinterpret_cast<uintptr_t>(grad_dev) | reinterpret_cast<uintptr_t>(out_dev) |
                     reinterpret_cast<uintptr_t>(recv_dev)) % 16 == 0;
    if (dtype == DYNB_F32) {
        if (al && row_bytes % 16 == 0) {
            const int64_t q = row_bytes / 16;
            unpack_add_rows_kernel<float, float4, 4><<<grid_for(n_local * q), 256, 0, s>>>(
                static_cast<const float4*>(grad_dev), n_local, q, static_cast<const float4*>(recv_dev), inv_offsets_dev,
                inv_entries_dev, static_cast<float4*>(out_dev));
        } else {
            unpack_add_rows_kernel<float, float, 1><<<grid_for(n_local * feature_dim), 256, 0, s>>>(
                static_cast<const float*>(grad_dev), n_local, feature_dim, static_cast<const float*>(recv_dev), inv_offsets_dev,
                inv_entries_dev, static_cast<float*>(out_dev));
        }
    } else {
        if (al && row_bytes % 16 == 0) {
            const int64_t q = row_bytes / 16;
            unpack_add_rows_kernel<double, double2, 2><<<grid_for(n_local * q), 256, 0, s>>>(
                static_cast<const double2*>(grad_dev), n_local, q, static_cast<const double2*>(recv_dev), inv_offsets_dev,
                inv_entries_dev, static_cast<double2*>(out_dev));
        } else {
            unpack_add_rows_kernel<double, double, 1><<<grid_for(n_local * feature_dim), 256, 0, s>>>(
                static_cast<const double*>(grad_dev), n_local, feature_dim, static_cast<const double*>(recv_dev), inv_offsets_dev,
                inv_entries_dev, static_cast<double*>(out_dev));
        }
    }
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

// ------------------------------------------------------------------------------------------ peer memory
// These four are the only calls of the library that allocate, free or map device memory.
extern "C" int dynb_ipc_alloc(int64_t bytes, void** ptr_out)
{
    if (bytes <= 0 || ptr_out == nullptr) return fail_arg("bad arguments");
    void* p = nullptr;
    DYNB_CUDA_OK(cudaMalloc(&p, (size_t)bytes));
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    if (e != cudaSuccess) { cudaFree(p); return fail_cuda(e, "cudaMemset"); }
    DYNB_CUDA_OK(cudaDeviceSynchronize());
    *ptr_out = p;
    return DYNB_OK;
}

extern "C" int dynb_ipc_free(void* ptr)
{
    if (ptr == nullptr) return DYNB_OK;
    DYNB_CUDA_OK(cudaFree(ptr));
    return DYNB_OK;
}

extern "C" int dynb_ipc_export(void* ptr, uint8_t* handle64_out)
{
    if (ptr == nullptr || handle64_out == nullptr) return fail_arg("null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    cudaIpcMemHandle_t h;
    DYNB_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle64_out, &h, 64);
    return DYNB_OK;
}

extern "C" int dynb_ipc_open(const uint8_t* handle64, void** ptr_out)
{
    if (handle64 == nullptr || ptr_out == nullptr) return fail_arg("null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    DYNB_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return DYNB_OK;
}

extern "C" int dynb_ipc_close(void* ptr)
{
    if (ptr == nullptr) return DYNB_OK;
    DYNB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return DYNB_OK;
}

extern "C" int dynb_copy_async(void* dst_dev, const void* src_dev, int64_t bytes, void* stream)
{
    if (bytes < 0) return fail_arg("bad arguments");
    if (bytes == 0) return DYNB_OK;
    DYNB_CUDA_OK(cudaMemcpyAsync(dst_dev, src_dev, (size_t)bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return DYNB_OK;
}

extern "C" int dynb_fill_zero(void* dst_dev, int64_t bytes, void* stream)
{
    if (bytes < 0) return fail_arg("bad arguments");
    if (bytes == 0) return DYNB_OK;
    if (dst_dev == nullptr) return fail_arg("null pointer");
    DYNB_CUDA_OK(cudaMemsetAsync(dst_dev, 0, (size_t)bytes, static_cast<cudaStream_t>(stream)));
    return DYNB_OK;
}

extern "C" int dynb_enable_peer_access(int peer_device)
{
    int dev = 0;
    DYNB_CUDA_OK(cudaGetDevice(&dev));
    if (peer_device == dev) return DYNB_OK;
    int can = 0;
    DYNB_CUDA_OK(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    if (!can) return fail_arg("peer access between these devices is not possible");
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return DYNB_OK; }
    DYNB_CUDA_OK(e);
    return DYNB_OK;
}
