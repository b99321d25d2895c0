"""CPU tests: the oracle is pinned against vectors produced by the REFERENCE's own CUDA kernels
(tests/golden/reference_vectors.npz, made by tests/golden/make_golden.py) and against the closed-form
cases the reference's tests assert."""

import importlib.util
import os

import numpy as np
import pytest

from oracle import cpu_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(mg)
G = np.load(os.path.join(HERE, "golden", "reference_vectors.npz"))


@pytest.mark.parametrize("name", sorted(mg.cases().keys()))
def test_radius_graph_matches_reference_vectors(name):
    pos, cell, pbc, r, targets = mg.cases()[name]
    g = O.radius_graph(pos, cell, pbc, r, targets)
    mine = O.canonical_edges(g["src"], g["dst"], g["shift"])
    ref = G[f"rg_{name}_edges"].astype(np.int64)
    assert mine.shape == ref.shape
    assert (mine == ref).all()
    np.testing.assert_array_equal(g["counts"], G[f"rg_{name}_counts"])


def test_known_answers():
    g = O.radius_graph(np.array([[2.5, 2.5, 2.5]], np.float32), np.eye(3, dtype=np.float32) * 5, [1, 1, 1], 6.0)
    assert g["E"] == 6 and (g["src"] == 0).all() and (g["dst"] == 0).all()
    assert not (np.abs(g["shift"]).sum(axis=1) == 0).any()
    assert sorted(map(tuple, g["shift"].tolist())) == sorted([(1, 0, 0), (-1, 0, 0), (0, 1, 0), (0, -1, 0), (0, 0, 1), (0, 0, -1)])
    g = O.radius_graph(np.array([[5, 5, 5]], np.float32), np.eye(3, dtype=np.float32) * 10, [0, 0, 0], 5.0)
    assert g["E"] == 0
    g = O.radius_graph(np.zeros((0, 3), np.float32), np.eye(3, dtype=np.float32), [1, 1, 1], 5.0)
    assert g["E"] == 0 and g["counts"].shape == (0,)


def test_radius_graph_agrees_with_kdtree_on_fcc():
    from scipy.spatial import cKDTree

    from dynamis_b200 import synthetic

    pos, cell, pbc, r = synthetic.fcc_copper(8)
    g = O.radius_graph(pos, cell, pbc, r)
    L = float(cell[0, 0])
    pw = np.mod(pos.astype(np.float64), L)
    pw[pw >= L] -= L
    pairs = cKDTree(pw, boxsize=L).query_pairs(r, output_type="ndarray")
    assert abs(g["E"] - 2 * len(pairs)) <= 4  # only pairs within an ulp of the cutoff may differ
    # edge vector convention: pos[src] + shift @ cell - pos[dst] has length <= r
    vec = pos[g["src"]].astype(np.float64) + g["shift"] @ cell.astype(np.float64) - pos[g["dst"]].astype(np.float64)
    d = np.linalg.norm(vec, axis=1)
    assert d.max() <= r * (1 + 1e-5) and d.min() > 1e-4
    np.testing.assert_allclose(d * d, g["d2"], rtol=2e-5)


def test_float64_instantiation_is_symmetric_and_consistent():
    from dynamis_b200 import synthetic

    pos, cell, pbc, r = synthetic.triclinic_silicon(4, 4, 2)
    g = O.radius_graph(pos, cell, pbc, r)
    fwd = set(zip(g["src"].tolist(), g["dst"].tolist(), map(tuple, g["shift"].tolist())))
    for s, d, sh in list(fwd)[:2000]:
        assert (d, s, tuple(-x for x in sh)) in fwd
    vec = pos[g["src"]] + g["shift"] @ cell - pos[g["dst"]]
    np.testing.assert_allclose((vec * vec).sum(axis=1), g["d2"], rtol=1e-12)


@pytest.mark.parametrize("W", [2, 8, 13])
def test_sfc_labels_match_reference_vectors(W):
    pos, w = mg.sfc_case()
    np.testing.assert_array_equal(O.sfc_partition(pos, None, W, 0), G[f"sfc_morton_W{W}"].astype(np.int64))
    np.testing.assert_array_equal(O.sfc_partition(pos, w, W, 0), G[f"sfc_morton_weighted_W{W}"].astype(np.int64))
    np.testing.assert_array_equal(np.bincount(O.sfc_partition(pos, None, W, 1), minlength=W), G[f"sfc_hilbert_counts_W{W}"])


@pytest.mark.parametrize("W", [2, 3, 5, 8, 13])
def test_kdtree_labels_match_reference_vectors(W):
    """The numpy restatement of the KD-tree bisection against labels the reference's own CUDA kernels
    produced on a B200 (tests/golden/make_golden.py --kdtree)."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors_kdtree.npz")
    kd = np.load(path)
    pos, w = mg.kdtree_case()
    np.testing.assert_array_equal(O.kdtree_partition(pos, None, W), kd[f"kd_W{W}"].astype(np.int64))
    np.testing.assert_array_equal(O.kdtree_partition(pos, w, W), kd[f"kd_weighted_W{W}"].astype(np.int64))


def test_sfc_invariants():
    rng = np.random.default_rng(0)
    pos = (rng.random((1001, 3)) * 30).astype(np.float32)
    for W in (1, 3, 8, 2000):
        lab = O.sfc_partition(pos, None, W, 0)
        cnt = np.bincount(lab, minlength=W)
        assert cnt.sum() == 1001 and cnt.max() - cnt[cnt > 0].min() <= 1 and lab.min() >= 0 and lab.max() < W
    assert O.sfc_partition(pos[:1], None, 1, 0).tolist() == [0]


@pytest.mark.parametrize("rank", [0, 1, 2, 3])
def test_halo_maps_match_reference_vectors(rank):
    pos, cell, pid, W = mg.halo_case()
    n = pos.shape[0]
    g = O.radius_graph(pos, cell, [1, 1, 1], np.float32(6.5))
    m = O.build_halo_maps(g["src"], g["dst"], pid, rank, W)
    np.testing.assert_array_equal(m["send_offsets"], G[f"halo_r{rank}_send_offsets"])
    np.testing.assert_array_equal(m["send_local_indices"], G[f"halo_r{rank}_send_local"])
    np.testing.assert_array_equal(m["recv_offsets"], G[f"halo_r{rank}_recv_offsets"])
    np.testing.assert_array_equal(m["recv_atom_global"], G[f"halo_r{rank}_recv_atom"])
    np.testing.assert_array_equal(np.packbits(m["interior_mask"]), G[f"halo_r{rank}_interior"])
    # the same through the per-rank edge list (extract_halo_info restatement)
    mine = np.nonzero(pid == rank)[0]
    gr = O.radius_graph(pos, cell, [1, 1, 1], np.float32(6.5), mine)
    so, sl, ro, rg, im, ra = O.extract_halo_info(np.stack([gr["src"], gr["dst"]]), pid, mine, rank, W, n)
    np.testing.assert_array_equal(sl, m["send_local_indices"])
    np.testing.assert_array_equal(ra, m["recv_atom_global"])
    np.testing.assert_array_equal(im, m["interior_mask"])
    # filter to 6.0: digest of the reference's filtered edge set
    fe, fs = O.filter_edges_to_radius(np.stack([gr["src"], gr["dst"]]), gr["shift"].astype(np.float32), pos, cell, 6.0)
    assert tuple(int(v) for v in G[f"halo_r{rank}_filtered_digest"]) == O.edge_set_digest(fe[0], fe[1], fs)


def test_send_recv_symmetry():
    pos, cell, pid, W = mg.halo_case()
    g = O.radius_graph(pos, cell, [1, 1, 1], np.float32(6.5))
    maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
    send = np.array([m["send_offsets"][1:] - m["send_offsets"][:-1] for m in maps])
    recv = np.array([m["recv_offsets"][1:] - m["recv_offsets"][:-1] for m in maps])
    np.testing.assert_array_equal(send, recv.T)
    feats = [np.full((m["num_local"], 2), r * 100000.0) + np.arange(m["num_local"])[:, None] for r, m in enumerate(maps)]
    out = O.exchange_forward(feats, [m["send_offsets"] for m in maps], [m["send_local_indices"] for m in maps],
                             [m["recv_offsets"] for m in maps])
    for r, m in enumerate(maps):
        ghosts = out[r][m["num_local"]:, 0]
        owner = (ghosts // 100000).astype(int)
        assert (owner == pid[m["recv_atom_global"]]).all()


def test_integrator_oracle_analytic_cases():
    """The closed-form cases of the reference's integrator tests (dynamis_integrator/tests/test_verlet.py,
    test_euler.py): the oracle must reproduce them before the CUDA kernels are compared with it."""
    f32 = lambda rows: np.array(rows, dtype=np.float32)
    pos, vel, frc, mass = f32([[0, 0, 0]]), f32([[0, 0, 0]]), f32([[2, 0, 0]]), f32([1])
    O.integrator_step(1, pos, vel, frc, mass, None, 0.5)
    np.testing.assert_allclose(vel, [[0.5, 0, 0]]); np.testing.assert_allclose(pos, [[0.25, 0, 0]])
    O.integrator_step(2, None, vel, frc, mass, None, 0.5)
    np.testing.assert_allclose(vel, [[1.0, 0, 0]])
    pos, vel, frc, mass = f32([[0, 0, 0]]), f32([[0, 0, 0]]), f32([[4, 0, 0]]), f32([2])
    O.integrator_step(0, pos, vel, frc, mass, None, 0.25)
    np.testing.assert_allclose(vel, [[0.5, 0, 0]]); np.testing.assert_allclose(pos, [[0.125, 0, 0]])
    # Langevin, gamma = 0: the noise drops out and the half-steps are Verlet's
    rng = np.random.default_rng(3)
    p, v, f = (rng.normal(size=(50, 3)).astype(np.float32) for _ in range(3))
    m = (rng.random(50) + 1).astype(np.float32); nz = rng.normal(size=(50, 3)).astype(np.float32)
    p2, v2 = p.copy(), v.copy()
    O.integrator_step(3, p, v, f, m, nz, 0.5, 0.0, 0.0257)
    O.integrator_step(1, p2, v2, f, m, None, 0.5)
    np.testing.assert_allclose(p, p2, rtol=1e-6); np.testing.assert_allclose(v, v2, rtol=1e-6)
    # drift word: bit 0 reach >= threshold, bit 1 displacement > threshold
    cur, ref = f32([[1, 0, 0], [0, 0, 0]]), f32([[0, 0, 0], [0, 0, 0]])
    vv, pv = f32([[0, 0, 0], [0, 0, 0]]), f32([[0, 0, 0], [0, 0, 0]])
    assert O.drift_flag(cur, ref, vv, pv.copy(), 0.5, 2.0) == 0
    assert O.drift_flag(cur, ref, vv, pv.copy(), 0.5, 1.0) == 1
    assert O.drift_flag(cur, ref, vv, pv.copy(), 0.5, 0.5) == 3
