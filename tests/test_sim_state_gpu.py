"""SimState (repartition, halo-only rebuild, drift watchdog) on one GPU, world size 1; the multi-rank
path runs under torchrun in test_multi_gpu.py.  The drift word is compared with the reference's formula
(dynamis/src/dynamis/simulatorState.py:257-293) evaluated with torch ops."""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def _system(n, L, dev, seed=0):
    rng = np.random.default_rng(seed)
    st = D.MolecularInfo()
    st.num_atoms = n
    st.atom_positions = torch.as_tensor((rng.random((n, 3)) * L).astype(np.float32), device=dev)
    st.atom_velocities = torch.as_tensor(rng.normal(0, 0.05, (n, 3)).astype(np.float32), device=dev)
    st.atom_types = torch.zeros(n, dtype=torch.int64, device=dev)
    st.atom_vertex_numbers = torch.arange(n, dtype=torch.int64, device=dev)
    cfg = D.SimulationConfig()
    cfg.cutoff, cfg.ghost_cutoff_buffer = 5.0, 0.5
    cfg.cell = torch.eye(3) * L
    cfg.pbc = torch.tensor([True, True, True])
    return st, cfg


def test_scatter_rows_matches_index_put(cuda):
    g = torch.Generator().manual_seed(1)
    for F, dt in ((3, torch.float32), (6, torch.float32), (4, torch.float64), (1, torch.int64)):
        rows = (torch.rand(5000, F, generator=g) * 100).to(dt).to(cuda)
        idx = torch.randperm(9000, generator=g)[:5000].to(cuda)
        out = torch.zeros(9000, F, dtype=dt, device=cuda)
        ref = out.clone()
        ref[idx] = rows
        D.scatter_rows(rows, idx, out)
        assert torch.equal(out, ref)


def _reference_drift_word(cur, ref, vel, prev, thr, dt):
    disp = (cur - ref).norm(dim=1)
    reach = disp + dt * (vel.norm(dim=1) + (vel - prev).norm(dim=1))
    return int(reach.max() >= thr) * 1 + int(disp.max() > thr) * 2


def test_drift_flag_matches_reference_formula(cuda):
    st, cfg = _system(20_000, 60.0, cuda, 3)
    env = D.DistEnvironment()
    env.global_rank, env.world_size, env.local_rank = 0, 1, 0
    s = D.SimState(st, D.SFCPartitioner(), cfg, env, device=cuda)
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    ref_pos = s.pos.clone()
    prev = s.vel.clone()
    for step, scale in enumerate((0.0, 0.1, 0.2, 0.26, 0.4)):
        s.pos.copy_(ref_pos + scale * torch.tensor([1.0, 0.0, 0.0], device=cuda))
        s.vel.mul_(1.1)
        want = _reference_drift_word(s.pos, ref_pos, s.vel, prev, 0.25, 0.5)
        s.write_local_drift_flag(flag, 0.25, 0.5)
        assert int(flag.item()) == want, (step, scale, int(flag.item()), want)
        prev = s.vel.clone()
    assert want == 3


def test_repartition_world_size_1(cuda):
    st, cfg = _system(6000, 44.0, cuda, 5)
    env = D.DistEnvironment()
    env.global_rank, env.world_size, env.local_rank = 0, 1, 0
    s = D.SimState(st, D.SFCPartitioner(), cfg, env, device=cuda)
    assert s.pos.shape == (6000, 3) and s.local_partition_info.send_offsets.tolist() == [0, 0]
    moved = s.pos + 0.3
    s.pos.copy_(moved)
    s.sync_positions_and_rebuild_halo()
    assert torch.equal(s._state.global_molecular_info.atom_positions[s.local_partition_info.partition_indices], moved)
    s.pos.add_(0.2)
    s.sync_and_repartition()
    assert torch.allclose(s.pos, moved + 0.2) and s.local_partition_info.interior_mask.all()
