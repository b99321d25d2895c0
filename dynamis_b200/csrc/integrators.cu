// Integrator steps for B200 (sm_100a), optionally fused with the drift word.
//
// Replaces the reference's integrator kernels (dynamis_integrator/src/csrc/euler_integrator.cu:9-26,
// verlet_integrator.cu:9-36, langevin_integrator.cu:9-52).  The per-component arithmetic is written with
// the same expression shapes, so that the compiler forms the same multiply-adds:
//   Euler        v += (f / m) * dt;               x += v * dt
//   Verlet 1     v += 0.5f * (f / m) * dt;        x += v * dt
//   Verlet 2     v += 0.5f * (f / m) * dt
//   Langevin 1   v = v * c1 + 0.5f * (f / m) * dt + c2 * noise;   x += v * dt
//   Langevin 2   v = (v + 0.5f * (f / m) * dt + c2 * noise) * c3
//   with c1 = 1 - 0.5 gamma dt, c2 = sqrt(gamma kT dt / m), c3 = 1 / (1 + 0.5 gamma dt).
// One thread owns one atom (three components), which lets the position-updating steps also produce the
// drift word of SimState.write_local_drift_flag (dynamis/src/dynamis/simulatorState.py:257-293) in the
// same pass over the state: the new positions and velocities are still in registers, so the watchdog
// costs the reference positions and the previous velocities (24 B/atom) instead of a second full pass.

#include "common.cuh"

namespace dynb {

enum { INT_EULER = 0, INT_VERLET1 = 1, INT_VERLET2 = 2, INT_LANGEVIN1 = 3, INT_LANGEVIN2 = 4 };

struct DriftArgs {
    const float* ref;     // [n,3] positions at the last rebuild
    float* prev_vel;      // [n,3] velocities of the previous step, overwritten
    uint32_t* state;      // 3 words, zero between calls
    int32_t* flag;        // the 2-bit word
    float threshold;
};

template <int KIND, bool DRIFT>
__global__ void __launch_bounds__(256)
integrate_kernel(float* __restrict__ pos, float* __restrict__ vel, const float* __restrict__ frc,
                 const float* __restrict__ mass, const float* __restrict__ noise, int64_t n, float dt, float gamma,
                 float kT, DriftArgs da)
{
    float reach = 0.0f, disp = 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float m = mass[i];
        float xn[3], vn[3];
#pragma unroll
        for (int k = 0; k < 3; k++) {
            const int64_t idx = 3 * i + k;
            float v = vel[idx];
            const float f = frc[idx];
            if (KIND == INT_EULER) {
                v += (f / m) * dt;
            } else if (KIND == INT_VERLET1 || KIND == INT_VERLET2) {
                v += 0.5f * (f / m) * dt;
            } else if (KIND == INT_LANGEVIN1) {
                const float c1 = 1.0f - 0.5f * gamma * dt;
                const float c2 = sqrtf(gamma * kT * dt / m);
                v = v * c1 + 0.5f * (f / m) * dt + c2 * noise[idx];
            } else {
                const float c3 = 1.0f / (1.0f + 0.5f * gamma * dt);
                const float c2 = sqrtf(gamma * kT * dt / m);
                v = (v + 0.5f * (f / m) * dt + c2 * noise[idx]) * c3;
            }
            vel[idx] = v;
            vn[k] = v;
            if (KIND == INT_EULER || KIND == INT_VERLET1 || KIND == INT_LANGEVIN1) {
                float x = pos[idx];
                x += v * dt;
                pos[idx] = x;
                xn[k] = x;
            } else {
                xn[k] = 0.0f;
            }
        }
        if (DRIFT) {
            // same expressions as drift_flag_kernel (state_ops.cu)
            const float dx = xn[0] - da.ref[3 * i], dy = xn[1] - da.ref[3 * i + 1], dz = xn[2] - da.ref[3 * i + 2];
            const float vx = vn[0], vy = vn[1], vz = vn[2];
            const float ax = vx - da.prev_vel[3 * i], ay = vy - da.prev_vel[3 * i + 1], az = vz - da.prev_vel[3 * i + 2];
            const float d = sqrtf(dx * dx + dy * dy + dz * dz);
            const float r = d + dt * (sqrtf(vx * vx + vy * vy + vz * vz) + sqrtf(ax * ax + ay * ay + az * az));
            disp = fmaxf(disp, d);
            reach = fmaxf(reach, r);
            da.prev_vel[3 * i] = vx; da.prev_vel[3 * i + 1] = vy; da.prev_vel[3 * i + 2] = vz;
        }
    }
    if (!DRIFT) return;
    // block maxima -> two atomics per block; the block that arrives last publishes the word and leaves
    // the state words zero for the next call (no block waits for another)
    __shared__ uint32_t sm[2][8];
    uint32_t rb = __float_as_uint(reach), db = __float_as_uint(disp);  // non-negative floats order like their bits
    rb = __reduce_max_sync(0xffffffffu, rb);
    db = __reduce_max_sync(0xffffffffu, db);
    if ((threadIdx.x & 31) == 0) { sm[0][threadIdx.x >> 5] = rb; sm[1][threadIdx.x >> 5] = db; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 0; w < 8; w++) { rb = max(rb, sm[0][w]); db = max(db, sm[1][w]); }
        atomicMax(&da.state[0], rb);
        atomicMax(&da.state[1], db);
        __threadfence();
        const uint32_t done = atomicAdd(&da.state[2], 1u);
        if (done == gridDim.x - 1) {
            __threadfence();
            const float R = __uint_as_float(atomicExch(&da.state[0], 0u));
            const float D = __uint_as_float(atomicExch(&da.state[1], 0u));
            da.state[2] = 0;
            *da.flag = ((R >= da.threshold) ? 1 : 0) + ((D > da.threshold) ? 2 : 0);
        }
    }
}

template <int KIND>
static int launch_integrator(float* pos, float* vel, const float* frc, const float* mass, const float* noise, int64_t n,
                             float dt, float gamma, float kT, const DriftArgs* da, cudaStream_t s)
{
    const unsigned g = (unsigned)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)sm_count_cached() * 8));
    if (da != nullptr) integrate_kernel<KIND, true><<<g, 256, 0, s>>>(pos, vel, frc, mass, noise, n, dt, gamma, kT, *da);
    else integrate_kernel<KIND, false><<<g, 256, 0, s>>>(pos, vel, frc, mass, noise, n, dt, gamma, kT, DriftArgs{});
    DYNB_CUDA_OK(cudaGetLastError());
    return DYNB_OK;
}

}  // namespace dynb

using namespace dynb;

extern "C" int dynb_integrator_step(int kind, float* pos_dev, float* vel_dev, const float* frc_dev, const float* mass_dev,
                                    const float* noise_dev, int64_t n_atoms, double dt, double gamma, double kT,
                                    const float* drift_ref_dev, float* drift_prev_vel_dev, double drift_threshold,
                                    uint32_t* drift_state_dev, int32_t* drift_flag_dev, void* stream)
{
    if (kind < INT_EULER || kind > INT_LANGEVIN2) return fail_arg("kind must be 0 (Euler), 1/2 (Verlet half-steps) or 3/4 (Langevin half-steps)");
    if (n_atoms < 0) return fail_arg("n_atoms must be non-negative");
    const bool moves = (kind == INT_EULER || kind == INT_VERLET1 || kind == INT_LANGEVIN1);
    const bool langevin = (kind == INT_LANGEVIN1 || kind == INT_LANGEVIN2);
    const bool drift = drift_flag_dev != nullptr;
    if (drift && !moves) return fail_arg("the drift word can only ride on a step that moves the positions");
    if (drift && (drift_ref_dev == nullptr || drift_prev_vel_dev == nullptr || drift_state_dev == nullptr))
        return fail_arg("drift word requested: reference positions, previous velocities and state words are required");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_atoms == 0) {
        if (drift) DYNB_CUDA_OK(cudaMemsetAsync(drift_flag_dev, 0, 4, s));
        return DYNB_OK;
    }
    if (vel_dev == nullptr || frc_dev == nullptr || mass_dev == nullptr || (moves && pos_dev == nullptr)) return fail_arg("null pointer");
    if (langevin && noise_dev == nullptr) return fail_arg("Langevin steps need a noise array");
    DriftArgs da{drift_ref_dev, drift_prev_vel_dev, drift_state_dev, drift_flag_dev, (float)drift_threshold};
    const DriftArgs* dp = drift ? &da : nullptr;
    const float fdt = (float)dt, fg = (float)gamma, fkT = (float)kT;
    switch (kind) {
        case INT_EULER: return launch_integrator<INT_EULER>(pos_dev, vel_dev, frc_dev, mass_dev, noise_dev, n_atoms, fdt, fg, fkT, dp, s);
        case INT_VERLET1: return launch_integrator<INT_VERLET1>(pos_dev, vel_dev, frc_dev, mass_dev, noise_dev, n_atoms, fdt, fg, fkT, dp, s);
        case INT_VERLET2: return launch_integrator<INT_VERLET2>(pos_dev, vel_dev, frc_dev, mass_dev, noise_dev, n_atoms, fdt, fg, fkT, dp, s);
        case INT_LANGEVIN1: return launch_integrator<INT_LANGEVIN1>(pos_dev, vel_dev, frc_dev, mass_dev, noise_dev, n_atoms, fdt, fg, fkT, dp, s);
        default: return launch_integrator<INT_LANGEVIN2>(pos_dev, vel_dev, frc_dev, mass_dev, noise_dev, n_atoms, fdt, fg, fkT, dp, s);
    }
}
