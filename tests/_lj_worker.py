"""Worker for test_lj_caller_gpu.py (torchrun, one rank per GPU, also with a single rank).

A Lennard-Jones model written the way the reference's dependency-free caller is written
(dynamis_model/src/dynamis_model/empirical/lj_potential_model.py:14-175): it imports ``dynamis_state`` and
``dynamis_model`` — here resolved to dynamis_b200's drop-in packages —, pushes positions and atom types
through ``FeaturePushToExchange`` / ``GPUDirectExchanger``, builds the graph with
``radius_graph_pbc_cuda`` and differentiates the energy back through the exchange.  Energies and forces
are compared with a dense all-pairs evaluation of the same formula in float64."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import dynamis_b200  # noqa: E402

dynamis_b200.install_shim()
from dynamis_model import DynamisModel  # noqa: E402
from dynamis_model.comm.exchanger import GPUDirectExchanger  # noqa: E402
from dynamis_model.comm.feature_push import FeaturePushToExchange  # noqa: E402
from dynamis_state import (  # noqa: E402
    DynamisState,
    MolecularInfo,
    SFCPartitioner,
    SimulationConfig,
    TorchDistEnv,
    radius_graph_pbc_cuda,
)


def lj_energy(atom_types, positions, edge_index, epsilon, sigma, n_local):
    i, j = edge_index[0], edge_index[1]
    keep = i < n_local                     # every pair is seen once from each side: halve at the end
    i, j = i[keep], j[keep]
    d = torch.linalg.norm(positions[i] - positions[j], dim=1).clamp(min=1e-6)
    far = d > 2.5                          # closer pairs count as bonded
    i, j, d = i[far], j[far], d[far]
    s = (sigma[atom_types[i]] + sigma[atom_types[j]]) / 2.0
    e = torch.sqrt(epsilon[atom_types[i]] * epsilon[atom_types[j]])
    sr6 = (s / d) ** 6
    return (4 * e * (sr6 ** 2 - sr6)).sum() / 2.0


class LJ(DynamisModel):
    def __init__(self, epsilon, sigma):
        super().__init__()
        self.epsilon, self.sigma = epsilon, sigma
        self.position_exchanger = GPUDirectExchanger()
        self.atom_type_exchanger = GPUDirectExchanger()

    def initialize_buffers(self, partition_info, device):
        self.position_exchanger.setup_exchanger(feature_dim=3, partition_info=partition_info, device=device)
        self.atom_type_exchanger.setup_exchanger(feature_dim=1, partition_info=partition_info, device=device)

    def __call__(self, state: DynamisState):
        local = state.local_molecular_info.atom_positions.clone().detach().requires_grad_(True)
        positions = FeaturePushToExchange.apply(local, state, self.position_exchanger)
        with torch.no_grad():
            types = FeaturePushToExchange.apply(state.local_molecular_info.atom_types.float().unsqueeze(1), state,
                                                self.atom_type_exchanger).long().reshape(-1)
            cfg = state.sim_config
            data = type("Data", (object,), {"pos": positions, "cell": cfg.cell.unsqueeze(0), "natoms": [positions.shape[0]],
                                            "pbc": cfg.pbc})()
            edge_index, _, _ = radius_graph_pbc_cuda(data=data, radius=cfg.cutoff, max_num_neighbors_threshold=0,
                                                     enforce_max_neighbors_strictly=False)
        energy = lj_energy(types, positions, edge_index, self.epsilon, self.sigma, local.shape[0])
        energy.backward()
        return energy.detach(), -local.grad.detach()


def dense(pos, types, L, rc, epsilon, sigma):
    """All pairs in float64: a pair is an edge when its minimum-image distance is within the cutoff (and not
    zero); the model then uses the plain difference of the stored positions, as the caller above does."""
    p = pos.double().requires_grad_(True)
    dr = p[:, None, :] - p[None, :, :]
    mi = dr - L * torch.round(dr.detach() / L)
    dmin = torch.linalg.norm(mi.detach(), dim=2)
    edge = (dmin <= rc) & (dmin * dmin > 1e-8)
    d = torch.linalg.norm(dr + torch.eye(p.shape[0], device=p.device, dtype=p.dtype)[:, :, None], dim=2).clamp(min=1e-6)
    use = edge & (d > 2.5)
    s = (sigma[types][:, None] + sigma[types][None, :]).double() / 2.0
    e = torch.sqrt(epsilon[types][:, None] * epsilon[types][None, :]).double()
    sr6 = torch.where(use, (s / d) ** 6, torch.zeros_like(d))
    energy = (4 * e * (sr6 ** 2 - sr6)).sum() / 2.0
    energy.backward()
    return energy.detach(), -p.grad.detach()


def main():
    env = TorchDistEnv(is_distributed=True)
    dev, rank, W = env.device, env.global_rank, env.world_size
    rng = np.random.default_rng(17)
    a, nc = 5.26, 10                                     # fcc argon, 4000 atoms, L = 52.6
    basis = np.array([[0, 0, 0], [.5, .5, 0], [.5, 0, .5], [0, .5, .5]])
    cells = np.stack(np.meshgrid(*[np.arange(nc)] * 3, indexing="ij"), -1).reshape(-1, 3)
    pos = ((cells[:, None, :] + basis[None]).reshape(-1, 3) * a + rng.normal(0, 0.12, (4 * nc ** 3, 3))).astype(np.float32)
    L, rc = a * nc, 8.0
    n = pos.shape[0]
    types = rng.integers(0, 2, n)
    eps = torch.tensor([0.0104, 0.0140], device=dev)
    sig = torch.tensor([3.40, 3.10], device=dev)
    tp, tt = torch.as_tensor(pos, device=dev), torch.as_tensor(types, device=dev)

    mol = MolecularInfo()
    mol.num_atoms, mol.atom_positions, mol.atom_types = n, tp, tt
    mol.atom_vertex_numbers = torch.arange(n, dtype=torch.int64, device=dev)
    cfg = SimulationConfig()
    cfg.cutoff, cfg.ghost_cutoff_buffer = rc, 0.5
    cfg.cell, cfg.pbc = torch.eye(3, device=dev) * L, torch.tensor([True, True, True], device=dev)
    part = SFCPartitioner()
    info = part.partition(mol, env.dist_env)
    part.build_halo_maps(info, mol, env.dist_env, cfg)
    state = DynamisState()
    loc = MolecularInfo()
    loc.atom_positions, loc.atom_types = tp[info.partition_indices].contiguous(), tt[info.partition_indices].contiguous()
    loc.num_atoms = int(info.partition_indices.numel())
    state.local_molecular_info, state.local_partition_info, state.sim_config = loc, info, cfg
    state.global_molecular_info = mol

    model = LJ(eps, sig)
    model.initialize_buffers(info, dev)
    for it in range(2):
        e_loc, f_loc = model(state)
    e_all = e_loc.clone()
    dist.all_reduce(e_all)
    forces = torch.zeros((n, 3), device=dev)
    forces[info.partition_indices] = f_loc
    dist.all_reduce(forces)

    e_ref, f_ref = dense(tp, tt, L, rc, eps, sig)
    rel_e = abs(float(e_all) - float(e_ref)) / abs(float(e_ref))
    err_f = float((forces.double() - f_ref).abs().max())
    scale = float(f_ref.abs().max())
    assert rel_e < 1e-5, f"energy {float(e_all)} vs dense {float(e_ref)}"
    assert err_f < 2e-5 * max(scale, 1.0), f"forces differ by {err_f} (largest component {scale})"
    for x in (model.position_exchanger, model.atom_type_exchanger):
        x.reset_buffers()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok  E = {float(e_all):.6f}  dense {float(e_ref):.6f}  max |dF| = {err_f:.2e}", flush=True)


if __name__ == "__main__":
    main()
