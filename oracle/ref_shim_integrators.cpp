// TEST INFRASTRUCTURE ONLY — exposes the reference's integrator steps as torch ops so that the GPU
// parity tests can run them next to ours on the same inputs.
//
// This file is ours; the implementations it forwards to are compiled, unmodified, from the
// reference's sources where they lie (see build_ref.py):
//   dynamis_integrator/src/csrc/euler_integrator.cu      EulerIntegrator::step
//   dynamis_integrator/src/csrc/verlet_integrator.cu     VerletIntegrator::halfstep1 / halfstep2
//   dynamis_integrator/src/csrc/langevin_integrator.cu   LangevinIntegrator::halfstep1 / halfstep2
// All five update their tensors in place.
#include "dynamis_integrator/integrator.hpp"
#include <torch/library.h>

static void ref_euler_step(at::Tensor pos, at::Tensor vel, at::Tensor frc, at::Tensor mass, double dt)
{
    dynamis_integrator::EulerIntegrator().step(pos, vel, frc, mass, (float)dt);
}
static void ref_verlet1(at::Tensor pos, at::Tensor vel, at::Tensor frc, at::Tensor mass, double dt)
{
    dynamis_integrator::VerletIntegrator().halfstep1(pos, vel, frc, mass, (float)dt);
}
static void ref_verlet2(at::Tensor vel, at::Tensor frc, at::Tensor mass, double dt)
{
    dynamis_integrator::VerletIntegrator().halfstep2(vel, frc, mass, (float)dt);
}
static void ref_langevin1(at::Tensor pos, at::Tensor vel, at::Tensor frc, at::Tensor mass, at::Tensor noise, double gamma,
                          double kT, double dt)
{
    dynamis_integrator::LangevinIntegrator().halfstep1(pos, vel, frc, mass, noise, (float)gamma, (float)kT, (float)dt);
}
static void ref_langevin2(at::Tensor vel, at::Tensor frc, at::Tensor mass, at::Tensor noise, double gamma, double kT, double dt)
{
    dynamis_integrator::LangevinIntegrator().halfstep2(vel, frc, mass, noise, (float)gamma, (float)kT, (float)dt);
}

TORCH_LIBRARY_FRAGMENT(dynamis_ref, m)
{
    m.def("euler_step(Tensor(a!) pos, Tensor(b!) vel, Tensor frc, Tensor mass, float dt) -> ()", &ref_euler_step);
    m.def("verlet_halfstep1(Tensor(a!) pos, Tensor(b!) vel, Tensor frc, Tensor mass, float dt) -> ()", &ref_verlet1);
    m.def("verlet_halfstep2(Tensor(a!) vel, Tensor frc, Tensor mass, float dt) -> ()", &ref_verlet2);
    m.def("langevin_halfstep1(Tensor(a!) pos, Tensor(b!) vel, Tensor frc, Tensor mass, Tensor noise, float gamma, float kT, "
          "float dt) -> ()", &ref_langevin1);
    m.def("langevin_halfstep2(Tensor(a!) vel, Tensor frc, Tensor mass, Tensor noise, float gamma, float kT, float dt) -> ()",
          &ref_langevin2);
}
