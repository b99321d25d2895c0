/*
 * TEST INFRASTRUCTURE ONLY — CPU oracle for the integrator steps and the drift word.
 *
 * Restates the per-component arithmetic of the reference's integrator kernels
 * (dynamis_integrator/src/csrc/euler_integrator.cu:18-24, verlet_integrator.cu:18-21 and :32-34,
 * langevin_integrator.cu:21-31 and :44-51) with every multiply-add the CUDA compiler forms from those
 * expressions written out as an explicit fmaf (built with -ffp-contract=off):
 *   a + b * c            -> fmaf(b, c, a)
 *   1 - a * b            -> fmaf(-a, b, 1)
 *   a * b + c * d + e*f  -> fmaf(e, f, fmaf(a, b, c * d))
 * Parity unpinned: the reference's integrator sources include a header that its build system
 * generates (dynamis_state/timing_config.hpp), so they cannot be compiled here; the known-answer
 * cases of its tests (dynamis_integrator/tests/test_verlet.py, test_euler.py, test_langevin.py) are
 * checked in tests/ instead.
 * The drift word follows dynamis/src/dynamis/simulatorState.py:257-293.
 */
#include <math.h>
#include <stdint.h>

/* kind: 0 Euler, 1/2 Verlet half-steps, 3/4 Langevin half-steps */
void orc_integrator_step(int kind, float *pos, float *vel, const float *frc, const float *mass, const float *noise,
                         int64_t n, float dt, float gamma, float kT)
{
    for (int64_t i = 0; i < n; i++) {
        const float m = mass[i];
        for (int k = 0; k < 3; k++) {
            const int64_t idx = 3 * i + k;
            float v = vel[idx];
            const float f = frc[idx];
            if (kind == 0) {
                v = fmaf(f / m, dt, v);
            } else if (kind == 1 || kind == 2) {
                v = fmaf(0.5f * (f / m), dt, v);
            } else if (kind == 3) {
                const float c1 = fmaf(-(0.5f * gamma), dt, 1.0f);
                const float c2 = sqrtf(gamma * kT * dt / m);
                v = fmaf(c2, noise[idx], fmaf(v, c1, (0.5f * (f / m)) * dt));
            } else {
                const float c3 = 1.0f / fmaf(0.5f * gamma, dt, 1.0f);
                const float c2 = sqrtf(gamma * kT * dt / m);
                v = fmaf(c2, noise[idx], fmaf(0.5f * (f / m), dt, v)) * c3;
            }
            vel[idx] = v;
            if (kind == 0 || kind == 1 || kind == 3) pos[idx] = fmaf(v, dt, pos[idx]);
        }
    }
}

/* bit 0: max_i(|x_i - ref_i| + dt (|v_i| + |v_i - vprev_i|)) >= threshold; bit 1: max_i |x_i - ref_i| > threshold;
 * prev_vel is overwritten with vel.  The sums of squares are the CUDA compiler's fmaf chains. */
int orc_drift_flag(const float *cur, const float *ref, const float *vel, float *prev_vel, int64_t n, float dt, float threshold)
{
    float reach = 0.0f, disp = 0.0f;
    for (int64_t i = 0; i < n; i++) {
        const float dx = cur[3 * i] - ref[3 * i], dy = cur[3 * i + 1] - ref[3 * i + 1], dz = cur[3 * i + 2] - ref[3 * i + 2];
        const float vx = vel[3 * i], vy = vel[3 * i + 1], vz = vel[3 * i + 2];
        const float ax = vx - prev_vel[3 * i], ay = vy - prev_vel[3 * i + 1], az = vz - prev_vel[3 * i + 2];
        const float d = sqrtf(fmaf(dz, dz, fmaf(dx, dx, dy * dy)));
        const float sv = sqrtf(fmaf(vz, vz, fmaf(vx, vx, vy * vy)));
        const float sa = sqrtf(fmaf(az, az, fmaf(ax, ax, ay * ay)));
        const float r = fmaf(dt, sv + sa, d);
        if (d > disp) disp = d;
        if (r > reach) reach = r;
        prev_vel[3 * i] = vx; prev_vel[3 * i + 1] = vy; prev_vel[3 * i + 2] = vz;
    }
    return ((reach >= threshold) ? 1 : 0) + ((disp > threshold) ? 2 : 0);
}
