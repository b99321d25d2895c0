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
// otherwise row i of the list is x[row_index[i]] (forward push).
template <typename V>
__global__ void __launch_bounds__(256)
push_rows_kernel(const V* __restrict__ x, int64_t q, const int64_t* __restrict__ row_index, int64_t src_row_base,
                 PushTable tab, int64_t total_rows)
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
        V* dst = reinterpret_cast<V*>(st[t].remote_ptr);
        dst[(st[t].remote_row_offset + (row - st[t].start)) * q + col] = x[src * q + col];
    }
    __threadfence_system();  // peer stores performed before this kernel's completion is signalled
}

// ------------------------------------------------------------------------------------------ signal / wait
__global__ void signal_peers_kernel(uint32_t* const* __restrict__ remote_flags, int n, uint32_t value)
{
    const int k = threadIdx.x;
    if (k < n && remote_flags[k] != nullptr) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote_flags[k]), "r"(value) : "memory");
    }
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Lane k waits until flags[k] >= value (wrap-safe compare) or the budget runs out.  On expiry it
// records 1 + k in *status (first expiry wins) and returns; nothing traps and nothing spins forever.
__global__ void wait_flags_kernel(const uint32_t* __restrict__ flags, const uint8_t* __restrict__ expect, int n,
                                  uint32_t value, unsigned long long budget_ns, uint32_t* __restrict__ status)
{
    const int k = threadIdx.x;
    if (k >= n || (expect != nullptr && !expect[k])) return;
    const unsigned long long t0 = globaltimer_ns();
    unsigned long long spins = 0;
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + k) : "memory");
        if ((int32_t)(v - value) >= 0) return;
        spins++;
        if ((spins & 63) == 0) {
            if (globaltimer_ns() - t0 > budget_ns || spins > (1ull << 34)) {
                atomicCAS(status, 0u, (uint32_t)(1 + k));
                return;
            }
        }
        __nanosleep(64);
    }
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

// The same sum restricted to the rows that receive something: out already holds grad (copied while the
// rows were still on their way), rows[] lists the local rows named by at least one send entry.
template <typename T, typename V, int VW>
__global__ void __launch_bounds__(256)
add_rows_listed_kernel(const int64_t* __restrict__ rows, int64_t n_rows, int64_t q, const V* __restrict__ recv,
                       const int64_t* __restrict__ inv_offsets, const uint32_t* __restrict__ inv_entries, V* __restrict__ out)
{
    const int64_t total = n_rows * q;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / q, col = i - r * q;
        const int64_t row = rows[r];
        V v = out[row * q + col];
        const int64_t b = inv_offsets[row], e = inv_offsets[row + 1];
        T* a = reinterpret_cast<T*>(&v);
        for (int64_t k = b; k < e; k++) {
            const V x = recv[(int64_t)inv_entries[k] * q + col];
            const T* xx = reinterpret_cast<const T*>(&x);
#pragma unroll
            for (int c = 0; c < VW; c++) a[c] += xx[c];
        }
        out[row * q + col] = v;
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

extern "C" int dynb_push_rows(const void* x_dev, int64_t row_bytes, const int64_t* row_index_dev, int64_t src_row_base,
                              const dynb_push_target* targets_dev, int n_targets, int64_t total_rows, int remote_align,
                              void* stream)
{
    if (row_bytes <= 0 || n_targets < 0 || n_targets > PUSH_MAX_TARGETS || total_rows < 0) return fail_arg("bad arguments");
    if (total_rows == 0 || n_targets == 0) return DYNB_OK;
    if (x_dev == nullptr || targets_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int vb = vec_bytes(row_bytes, x_dev, x_dev);
    if (remote_align < vb) vb = (remote_align >= 4 && row_bytes % 4 == 0) ? 4 : 1;
    const int64_t q = row_bytes / vb;
    PushTable tab{targets_dev, n_targets};
    const unsigned g = grid_for(total_rows * q);
    if (vb == 16) push_rows_kernel<uint4><<<g, 256, 0, s>>>(static_cast<const uint4*>(x_dev), q, row_index_dev, src_row_base, tab, total_rows);
    else if (vb == 4) push_rows_kernel<uint32_t><<<g, 256, 0, s>>>(static_cast<const uint32_t*>(x_dev), q, row_index_dev, src_row_base, tab, total_rows);
    else push_rows_kernel<uint8_t><<<g, 256, 0, s>>>(static_cast<const uint8_t*>(x_dev), q, row_index_dev, src_row_base, tab, total_rows);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_signal_peers(uint32_t* const* remote_flag_ptrs_dev, int n, uint32_t value, void* stream)
{
    if (n < 0 || n > 1024) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    signal_peers_kernel<<<1, ((n + 31) / 32) * 32, 0, static_cast<cudaStream_t>(stream)>>>(remote_flag_ptrs_dev, n, value);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_wait_flags(const uint32_t* flags_dev, const uint8_t* expect_dev, int n, uint32_t value, int64_t timeout_ns,
                               uint32_t* status_dev, void* stream)
{
    if (n < 0 || n > 1024 || timeout_ns <= 0 || status_dev == nullptr) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    wait_flags_kernel<<<1, ((n + 31) / 32) * 32, 0, static_cast<cudaStream_t>(stream)>>>(flags_dev, expect_dev, n, value,
                                                                                          (unsigned long long)timeout_ns, status_dev);
    DYNB_CUDA_OK(cudaGetLastError());
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

extern "C" int dynb_add_rows_listed(const int64_t* rows_dev, int64_t n_rows, int64_t feature_dim, int dtype, const void* recv_dev,
                                    const int64_t* inv_offsets_dev, const uint32_t* inv_entries_dev, void* out_dev, void* stream)
{
    if (n_rows < 0 || feature_dim <= 0) return fail_arg("bad arguments");
    if (dtype != DYNB_F32 && dtype != DYNB_F64) return fail_arg("dtype must be DYNB_F32 or DYNB_F64");
    if (n_rows == 0) return DYNB_OK;
    if (rows_dev == nullptr || out_dev == nullptr || inv_offsets_dev == nullptr || inv_entries_dev == nullptr || recv_dev == nullptr)
        return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t row_bytes = feature_dim * (dtype == DYNB_F64 ? 8 : 4);
    const bool al = (reinterpret_cast<uintptr_t>(out_dev) | reinterpret_cast<uintptr_t>(recv_dev)) % 16 == 0;
    if (dtype == DYNB_F32) {
        if (al && row_bytes % 16 == 0) {
            const int64_t q = row_bytes / 16;
            add_rows_listed_kernel<float, float4, 4><<<grid_for(n_rows * q), 256, 0, s>>>(
                rows_dev, n_rows, q, static_cast<const float4*>(recv_dev), inv_offsets_dev, inv_entries_dev, static_cast<float4*>(out_dev));
        } else {
            add_rows_listed_kernel<float, float, 1><<<grid_for(n_rows * feature_dim), 256, 0, s>>>(
                rows_dev, n_rows, feature_dim, static_cast<const float*>(recv_dev), inv_offsets_dev, inv_entries_dev, static_cast<float*>(out_dev));
        }
    } else {
        if (al && row_bytes % 16 == 0) {
            const int64_t q = row_bytes / 16;
            add_rows_listed_kernel<double, double2, 2><<<grid_for(n_rows * q), 256, 0, s>>>(
                rows_dev, n_rows, q, static_cast<const double2*>(recv_dev), inv_offsets_dev, inv_entries_dev, static_cast<double2*>(out_dev));
        } else {
            add_rows_listed_kernel<double, double, 1><<<grid_for(n_rows * feature_dim), 256, 0, s>>>(
                rows_dev, n_rows, feature_dim, static_cast<const double*>(recv_dev), inv_offsets_dev, inv_entries_dev, static_cast<double*>(out_dev));
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
