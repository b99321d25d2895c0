"""DistGraphBuilder on one GPU (world size 1): the refresh pass equals the oracle graph, the steady
pass equals the refresh pass, a small drift keeps the steady mode and a large one forces a refresh
(the reference's dynamis_state/tests/test_dist_graph_builder.py:537-622 schedule checks).  The
multi-rank behaviour is covered under torchrun in test_multi_gpu.py."""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from _util import assert_same_edges, canon_o, canon_t
from dynamis_b200.dist_graph_builder import BuildMode, DistGraphBuilder, cell_block_targets
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def test_refresh_and_steady_schedule(cuda):
    rng = np.random.default_rng(8)
    n, L = 3000, 36.0
    pos = (rng.random((n, 3)) * L).astype(np.float32)
    cell = (np.eye(3) * L).astype(np.float32)
    env = D.DistEnvironment()
    env.global_rank, env.world_size = 0, 1
    b = DistGraphBuilder(torch.as_tensor(cell, device=cuda), torch.tensor([True] * 3), 6.0, 0.5, env, refresh_interval=3)
    tp = torch.as_tensor(pos, device=cuda)
    g = O.radius_graph(pos, cell, [1, 1, 1], 6.0)
    r0 = b.build(tp)
    assert r0.mode == BuildMode.REFRESH
    assert_same_edges(canon_t(r0.edges_outer, r0.cell_shifts_outer), canon_o(g), "refresh")
    np.testing.assert_array_equal(r0.full_degrees.cpu().numpy(), g["counts"])
    assert r0.halo_info.send_offsets.tolist() == [0, 0] and r0.interior_mask.all()
    r1 = b.build(tp)
    assert r1.mode == BuildMode.STEADY
    assert_same_edges(canon_t(r1.edges_outer, r1.cell_shifts_outer), canon_o(g), "steady == refresh")
    small = tp + 0.1 * torch.tensor([1.0, 0.0, 0.0], device=cuda)
    assert b.build(small).mode == BuildMode.STEADY            # 0.1 A < skin / 2
    big = tp + 1.0 * torch.tensor([0.0, 1.0, 0.0], device=cuda)
    r3 = b.build(big)
    assert r3.mode == BuildMode.REFRESH                       # 1 A > skin / 2 forces a refresh
    b.reset()
    assert b.next_is_refresh


def test_cell_block_targets_cover_all_atoms(cuda):
    rng = np.random.default_rng(9)
    pos = torch.as_tensor((rng.random((5000, 3)) * 40.0).astype(np.float32), device=cuda)
    box = torch.tensor([40.0, 40.0, 40.0], device=cuda)
    got = torch.cat([cell_block_targets(pos, box, 6.5, r, 3) for r in range(3)])
    assert torch.equal(torch.sort(got).values, torch.arange(5000, device=cuda))
