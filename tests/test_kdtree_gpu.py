"""KD-tree partition (reference: dynamis_state/src/csrc/partition/kdtree_kernels.cu, kdtree_partitioner.cpp).

* labels equal the numpy oracle's for equal counts and for weights, powers of two and other W, repeated
  coordinates (ordered by atom index), all atoms on one point, fewer atoms than parts;
* labels equal those of the reference's own CUDA kernels, compiled from its sources, on inputs whose
  coordinates are distinct (its sort leaves ties open) and whose weight sums stay below 2**24 (its float32
  cumulative sum is exact there);
* KDTreePartitioner: the invariants the reference's tests check (ids in range, counts add up, every atom
  owned once, spatial locality of the halves), and the three calling modes.
"""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from dynamis_b200.state import DistEnvironment, MolecularInfo, SimulationConfig
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def _distinct_positions(n, seed, scale=10.0):
    """Every coordinate value occurs once per axis: a shuffled ramp plus sub-step jitter."""
    rng = np.random.default_rng(seed)
    pos = np.empty((n, 3), dtype=np.float32)
    for d in range(3):
        ramp = (np.arange(n, dtype=np.float64) + rng.random(n) * 0.5) * (scale / n)
        pos[:, d] = rng.permutation(ramp).astype(np.float32)
        assert np.unique(pos[:, d]).size == n
    return pos


@pytest.mark.parametrize("W", [1, 2, 3, 5, 8, 16, 37])
@pytest.mark.parametrize("weighted", [False, True])
def test_labels_match_oracle(cuda, W, weighted):
    rng = np.random.default_rng(300 + W)
    n = 20_011
    pos = (rng.random((n, 3)) * np.array([30.0, 10.0, 20.0])).astype(np.float32)
    pos[500:900, 0] = pos[500, 0]            # repeated coordinates along the first split axis
    w = rng.integers(0, 60, n).astype(np.int64) if weighted else None
    labels = D.kdtree_partition_labels(torch.as_tensor(pos, device=cuda), None if w is None else torch.as_tensor(w, device=cuda), W)
    np.testing.assert_array_equal(labels.cpu().numpy(), O.kdtree_partition(pos, w, W))


@pytest.mark.parametrize("W", [2, 7, 8, 64, 300])
def test_selection_and_sorted_paths_agree(cuda, W):
    """Equal-count cuts come from a selection (no sort); sorted_cuts takes the sorted path, which the
    weighted cuts always use.  Same labels on inputs with many repeated coordinates."""
    rng = np.random.default_rng(41 + W)
    pos = (rng.random((20_000, 3)) * 8.0).astype(np.float32)
    pos[:, 0] = np.round(pos[:, 0], 1)            # ~80 distinct values along x: long runs of ties
    pos[3000:3500] = pos[3000]
    tp = torch.as_tensor(pos, device=cuda)
    by_selection = D.kdtree_partition_labels(tp, None, W)
    by_sort = D.kdtree_partition_labels(tp, None, W, sorted_cuts=True)
    assert torch.equal(by_selection, by_sort)
    np.testing.assert_array_equal(by_selection.cpu().numpy(), O.kdtree_partition(pos, None, W))


def test_degenerate_inputs(cuda):
    one_point = np.full((1000, 3), 3.25, dtype=np.float32)
    for W in (2, 8):
        got = D.kdtree_partition_labels(torch.as_tensor(one_point, device=cuda), None, W).cpu().numpy()
        np.testing.assert_array_equal(got, O.kdtree_partition(one_point, None, W))
    few = (np.random.default_rng(1).random((3, 3)) * 5).astype(np.float32)
    got = D.kdtree_partition_labels(torch.as_tensor(few, device=cuda), None, 8).cpu().numpy()
    np.testing.assert_array_equal(got, O.kdtree_partition(few, None, 8))
    heavy = np.zeros(2000, dtype=np.int64); heavy[17] = 10_000     # one atom carries all the weight
    pos = (np.random.default_rng(2).random((2000, 3)) * 9).astype(np.float32)
    got = D.kdtree_partition_labels(torch.as_tensor(pos, device=cuda), torch.as_tensor(heavy, device=cuda), 4).cpu().numpy()
    np.testing.assert_array_equal(got, O.kdtree_partition(pos, heavy, 4))
    empty = D.kdtree_partition_labels(torch.empty((0, 3), device=cuda), None, 4)
    assert empty.shape == (0,)
    with pytest.raises(RuntimeError):
        D.kdtree_partition_labels(torch.as_tensor(pos, device=cuda).double(), None, 4)
    with pytest.raises(RuntimeError):
        D.kdtree_partition_labels(torch.as_tensor(pos, device=cuda), None, 0)


@pytest.mark.parametrize("W", [2, 4, 6, 8, 13])
@pytest.mark.parametrize("weighted", [False, True])
def test_labels_vs_reference_kernels(cuda, ref_ops, W, weighted):
    n = 30_000
    pos = _distinct_positions(n, 900 + W)
    w = np.random.default_rng(W).integers(1, 40, n).astype(np.int64) if weighted else None   # sums < 2**24
    tp = torch.as_tensor(pos, device=cuda)
    tw = None if w is None else torch.as_tensor(w, device=cuda)
    ours = D.kdtree_partition_labels(tp, tw, W)
    ref = ref_ops.kdtree_partition(tp, tw, W)
    assert torch.equal(ours, ref)


def _state(n, dev, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    st = MolecularInfo()
    st.num_atoms = n
    st.atom_vertex_numbers = torch.arange(n, dtype=torch.int64, device=dev)
    st.atom_positions = (torch.rand(n, 3, generator=g) * 10.0).to(dev)
    return st


def _env(rank, W):
    env = DistEnvironment()
    env.global_rank, env.world_size, env.local_rank, env.gpus_per_node, env.num_nodes = rank, W, rank, W, 1
    return env


def test_partitioner_invariants_and_modes(cuda):
    n, W = 4000, 4
    st = _state(n, cuda)
    owned = []
    for r in range(W):
        info = D.KDTreePartitioner().partition(st, _env(r, W))
        pid = info.partition_id
        assert int(pid.min()) >= 0 and int(pid.max()) < W
        assert int(info.atom_counts.sum()) == n and info.atom_counts.tolist() == [1000] * 4
        assert int(info.global_send_recv_matrix[r, r]) == info.partition_indices.numel() == 1000
        owned.append(info.partition_indices)
    assert torch.equal(torch.sort(torch.cat(owned)).values, torch.arange(n, device=cuda))
    # locality: the first cut is along the widest axis and separates the halves by coordinate
    pos = st.atom_positions
    ext = pos.max(0).values - pos.min(0).values
    ax = int(ext.argmax())
    left, right = pos[pid < 2, ax], pos[pid >= 2, ax]
    assert float(left.max()) <= float(right.min())
    # weighted by edge_counts
    st.edge_counts = torch.randint(1, 30, (n,), device=cuda)
    info_w = D.KDTreePartitioner().partition(st, _env(0, W))
    cost = torch.bincount(info_w.partition_id, weights=st.edge_counts.double(), minlength=W)
    assert float(cost.max()) <= 1.1 * float(cost.mean())
    np.testing.assert_array_equal(info_w.partition_id.cpu().numpy(),
                                  O.kdtree_partition(pos.cpu().numpy(), st.edge_counts.cpu().numpy(), W))
    # with a SimulationConfig: weights are the in-degrees at the cutoff, the graph is kept
    cfg = SimulationConfig()
    cfg.cutoff, cfg.ghost_cutoff_buffer = 1.5, 0.5
    cfg.cell = torch.eye(3) * 10.0
    cfg.pbc = torch.tensor([True, True, True])
    st.edge_counts = None
    info_g = D.KDTreePartitioner().partition(st, _env(1, W), cfg)
    deg = torch.bincount(info_g.edge_index[1], minlength=n)
    np.testing.assert_array_equal(info_g.partition_id.cpu().numpy(), O.kdtree_partition(pos.cpu().numpy(), deg.cpu().numpy(), W))
