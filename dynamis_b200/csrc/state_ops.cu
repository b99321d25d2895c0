// Per-repartition and per-step state kernels for B200 (sm_100a).
//
//   dynb_scatter_rows  out[idx[i], :] = rows[i, :]: puts the rows gathered from all ranks back into
//                      canonical atom order.  Replaces cat + argsort + gather of
//                      SimState.sync_and_repartition (dynamis/src/dynamis/simulatorState.py:172-183)
//                      and the per-rank index_put loop of sync_positions_and_rebuild_halo (:238-242).
//   dynb_drift_flag    the 2-bit drift word of SimState.write_local_drift_flag (:257-293) in one
//                      kernel instead of five reductions; also advances the velocity history.

#include "common.cuh"

namespace dynb {

template <typename V>
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const V* __restrict__ rows, int64_t q, const int64_t* __restrict__ idx, int64_t n, int64_t n_out,
                    V* __restrict__ out, uint32_t* __restrict__ bad)
{
    const int64_t total = n * q;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / q, col = i - row * q;
        const int64_t dst = idx[row];
        if (dst < 0 || dst >= n_out) { if (bad) atomicOr(bad, 1u); continue; }
        out[dst * q + col] = rows[i];
    }
}

// state[0] = max reach bits, state[1] = max displacement bits (non-negative floats order like their
// bit patterns), state[2] = blocks done.  The last block to finish writes the flag word and clears
// the state for the next call; no block waits for another.
__global__ void __launch_bounds__(256)
drift_flag_kernel(const float* __restrict__ cur, const float* __restrict__ ref, const float* __restrict__ vel,
                  float* __restrict__ prev_vel, int64_t n, float dt, float threshold, uint32_t* __restrict__ state,
                  int32_t* __restrict__ flag)
{
    float reach = 0.0f, disp = 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float dx = cur[3 * i] - ref[3 * i], dy = cur[3 * i + 1] - ref[3 * i + 1], dz = cur[3 * i + 2] - ref[3 * i + 2];
        const float vx = vel[3 * i], vy = vel[3 * i + 1], vz = vel[3 * i + 2];
        const float ax = vx - prev_vel[3 * i], ay = vy - prev_vel[3 * i + 1], az = vz - prev_vel[3 * i + 2];
        const float d = sqrtf(dx * dx + dy * dy + dz * dz);
        const float r = d + dt * (sqrtf(vx * vx + vy * vy + vz * vz) + sqrtf(ax * ax + ay * ay + az * az));
        disp = fmaxf(disp, d);
        reach = fmaxf(reach, r);
        prev_vel[3 * i] = vx; prev_vel[3 * i + 1] = vy; prev_vel[3 * i + 2] = vz;
    }
    __shared__ uint32_t sm[2][8];
    uint32_t rb = __float_as_uint(reach), db = __float_as_uint(disp);
    rb = __reduce_max_sync(0xffffffffu, rb);
    db = __reduce_max_sync(0xffffffffu, db);
    if ((threadIdx.x & 31) == 0) { sm[0][threadIdx.x >> 5] = rb; sm[1][threadIdx.x >> 5] = db; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) { rb = max(rb, sm[0][w]); db = max(db, sm[1][w]); }
        rb = max(rb, sm[0][0]); db = max(db, sm[1][0]);
        atomicMax(&state[0], rb);
        atomicMax(&state[1], db);
        __threadfence();
        const uint32_t done = atomicAdd(&state[2], 1u);
        if (done == gridDim.x - 1) {
            __threadfence();
            const float R = __uint_as_float(atomicExch(&state[0], 0u));
            const float D = __uint_as_float(atomicExch(&state[1], 0u));
            state[2] = 0;
            *flag = ((R >= threshold) ? 1 : 0) + ((D > threshold) ? 2 : 0);
        }
    }
}

}  // namespace dynb

using namespace dynb;

extern "C" int dynb_scatter_rows(const void* rows_dev, int64_t row_bytes, const int64_t* idx_dev, int64_t n, int64_t n_out,
                                 void* out_dev, uint32_t* bad_dev, void* stream)
{
    if (n < 0 || n_out < 0 || row_bytes <= 0) return fail_arg("bad arguments");
    if (n == 0) return DYNB_OK;
    if (rows_dev == nullptr || idx_dev == nullptr || out_dev == nullptr) return fail_arg("null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uintptr_t pa = reinterpret_cast<uintptr_t>(rows_dev), pb = reinterpret_cast<uintptr_t>(out_dev);
    int vb = 1;
    if (row_bytes % 16 == 0 && pa % 16 == 0 && pb % 16 == 0) vb = 16;
    else if (row_bytes % 4 == 0 && pa % 4 == 0 && pb % 4 == 0) vb = 4;
    const int64_t q = row_bytes / vb;
    const unsigned g = (unsigned)std::max<int64_t>(1, std::min<int64_t>((n * q + 255) / 256, (int64_t)sm_count_cached() * 16));
    if (vb == 16) scatter_rows_kernel<uint4><<<g, 256, 0, s>>>(static_cast<const uint4*>(rows_dev), q, idx_dev, n, n_out, static_cast<uint4*>(out_dev), bad_dev);
    else if (vb == 4) scatter_rows_kernel<uint32_t><<<g, 256, 0, s>>>(static_cast<const uint32_t*>(rows_dev), q, idx_dev, n, n_out, static_cast<uint32_t*>(out_dev), bad_dev);
    else scatter_rows_kernel<uint8_t><<<g, 256, 0, s>>>(static_cast<const uint8_t*>(rows_dev), q, idx_dev, n, n_out, static_cast<uint8_t*>(out_dev), bad_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

extern "C" int dynb_drift_flag(const float* cur_dev, const float* ref_dev, const float* vel_dev, float* prev_vel_dev, int64_t n,
                               double dt, double threshold, uint32_t* state_dev, int32_t* flag_dev, void* stream)
{
    if (n < 0 || state_dev == nullptr || flag_dev == nullptr) return fail_arg("bad arguments");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n == 0) { DYNB_CUDA_OK(cudaMemsetAsync(flag_dev, 0, 4, s)); return DYNB_OK; }
    if (cur_dev == nullptr || ref_dev == nullptr || vel_dev == nullptr || prev_vel_dev == nullptr) return fail_arg("null pointer");
    const unsigned g = (unsigned)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)sm_count_cached() * 4));
    drift_flag_kernel<<<g, 256, 0, s>>>(cur_dev, ref_dev, vel_dev, prev_vel_dev, n, (float)dt, (float)threshold, state_dev, flag_dev);
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}
