"""GPU parity tests of the radius graph: CUDA path (through the C ABI) vs the CPU oracle, and vs the
reference's own CUDA kernels when oracle/_ref was built.

Cases mirror the reference's dynamis_state/tests/test_radius_graph_pbc_cuda.py (cubic 8/100/1000
atoms, cutoff > box/2, triclinic, PBC on two axes only, no PBC, empty, single atom, wrapper) and
add target subsets, positions outside the cell, float64 and a cutoff-tie stress case.
Edge sets are compared bit-exactly after canonical sorting.
"""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from _util import assert_same_edges, canon_o, canon_t, digest_t
from dynamis_b200 import synthetic
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def _run_ours(pos, cell, pbc, r, dev, targets=None):
    import dynamis_b200 as D

    tp = torch.as_tensor(pos, device=dev)
    tc = torch.as_tensor(cell, device=dev)
    tb = torch.as_tensor(np.asarray(pbc, dtype=bool))
    tt = torch.as_tensor(targets, device=dev) if targets is not None else None
    return D.radius_graph_pbc_ex(tp, tc, tb, r, 0, False, tt)


def _check_vs_oracle(pos, cell, pbc, r, dev, targets=None, what=""):
    ei, cs, nni, counts = _run_ours(pos, cell, pbc, r, dev, targets)
    g = O.radius_graph(pos, cell, pbc, r, targets)
    assert int(nni.item()) == g["E"], f"{what}: E {int(nni.item())} vs oracle {g['E']}"
    assert ei.shape == (2, g["E"]) and cs.shape == (g["E"], 3)
    assert ei.dtype == torch.int64 and cs.dtype == torch.float32 and counts.dtype == torch.int32
    assert_same_edges(canon_t(ei, cs), canon_o(g), what)
    np.testing.assert_array_equal(counts.cpu().numpy(), g["counts"])
    return ei, cs, g


def _cubic(n, box, seed, dtype=np.float32):
    rng = np.random.default_rng(seed)
    pos = (rng.random((n, 3)) * box).astype(dtype)
    return pos, (np.eye(3) * box).astype(dtype), [True, True, True]


@pytest.mark.parametrize("n,box,r", [(8, 10.0, 3.0), (100, 20.0, 5.0), (1000, 30.0, 5.0), (20, 10.0, 4.0), (50, 15.0, 4.0)])
def test_cubic(cuda, n, box, r):
    pos, cell, pbc = _cubic(n, box, 42 + n)
    _check_vs_oracle(pos, cell, pbc, r, cuda, what=f"cubic{n}")


def test_dense_cells_long_candidate_lists(cuda):
    """Candidate lists far beyond the 512 records the count pass keeps hit bits for: the edge list is then
    written by the distance-recomputing writer, walking each list in several chunks; with distances
    requested that writer is used for every input.  Both must agree with the oracle and with each other."""
    pos, cell, pbc = _cubic(3000, 10.0, 91)          # 3 atoms / A^3, ~340 neighbours each
    ei, cs, g = _check_vs_oracle(pos, cell, pbc, 3.0, cuda, what="dense")
    assert g["E"] > 900_000
    out = D.radius_graph_pbc_with_dist(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), 3.0)
    assert_same_edges(canon_t(out[0], out[1]), canon_t(ei, cs), "dense, with distances")
    # a sparse case through both writers: same edge set (the order inside a target's run may differ)
    pos, cell, pbc = _cubic(5000, 40.0, 92)
    a = _run_ours(pos, cell, pbc, 5.0, cuda)
    b = D.radius_graph_pbc_with_dist(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), 5.0)
    assert_same_edges(canon_t(a[0], a[1]), canon_t(b[0], b[1]), "sparse, both writers")
    assert torch.equal(a[0][1], b[0][1])              # targets' runs are the same ranges


def test_cutoff_larger_than_half_box(cuda):
    pos, cell, pbc = _cubic(30, 8.0, 7)
    _check_vs_oracle(pos, cell, pbc, 6.0, cuda, what="multi-image")


def test_box_smaller_than_cutoff(cuda):
    # rep = 2..3 image layers per axis
    pos, cell, pbc = _cubic(5, 2.5, 8)
    _check_vs_oracle(pos, cell, pbc, 6.0, cuda, what="tiny box")


def test_triclinic(cuda):
    rng = np.random.default_rng(3)
    cell = np.array([[12.0, 0.0, 0.0], [2.5, 11.0, 0.0], [1.5, -2.0, 13.0]], np.float32)
    pos = (rng.random((400, 3)) @ cell.astype(np.float64)).astype(np.float32)
    _check_vs_oracle(pos, cell, [True, True, True], 5.0, cuda, what="triclinic")


def test_pbc_xy_only(cuda):
    pos, cell, _ = _cubic(300, 14.0, 11)
    _check_vs_oracle(pos, cell, [True, True, False], 4.5, cuda, what="pbc xy")


def test_no_pbc(cuda):
    pos, cell, _ = _cubic(300, 14.0, 12)
    _check_vs_oracle(pos, cell, [False, False, False], 4.5, cuda, what="no pbc")


def test_cluster_in_large_vacuum_box(cuda):
    rng = np.random.default_rng(13)
    pos = (rng.random((500, 3)) * 12.0 + 400.0).astype(np.float32)
    cell = (np.eye(3) * 1000.0).astype(np.float32)
    _check_vs_oracle(pos, cell, [False, False, False], 5.0, cuda, what="cluster")
    _check_vs_oracle(pos, cell, [True, True, True], 5.0, cuda, what="cluster pbc")


def test_positions_outside_cell(cuda):
    rng = np.random.default_rng(14)
    pos = ((rng.random((500, 3)) - 0.5) * 60.0).astype(np.float32)  # spans [-30, 30) in a 15 Å box
    cell = (np.eye(3) * 15.0).astype(np.float32)
    _check_vs_oracle(pos, cell, [True, True, True], 4.0, cuda, what="unwrapped")


def test_empty(cuda):
    import dynamis_b200 as D

    ei, cs, nni = D.radius_graph_pbc(torch.empty(0, 3, device=cuda), torch.eye(3, device=cuda),
                                     torch.tensor([True, True, True]), 5.0, 100, False)
    assert ei.shape == (2, 0) and cs.shape == (0, 3) and int(nni.item()) == 0


def test_single_atom_with_pbc(cuda):
    # reference known answer: 6 edges, all (0, 0), no zero shift
    import dynamis_b200 as D

    pos = torch.tensor([[2.5, 2.5, 2.5]], device=cuda)
    ei, cs, _ = D.radius_graph_pbc(pos, torch.eye(3, device=cuda) * 5.0, torch.tensor([True, True, True]), 6.0, 100, False)
    assert ei.size(1) == 6
    assert torch.all(ei == 0)
    assert not torch.any(cs.abs().sum(dim=1) == 0)


def test_single_atom_no_pbc(cuda):
    import dynamis_b200 as D

    pos = torch.tensor([[5.0, 5.0, 5.0]], device=cuda)
    ei, _, _ = D.radius_graph_pbc(pos, torch.eye(3, device=cuda) * 10.0, torch.tensor([False, False, False]), 5.0, 100, False)
    assert ei.size(1) == 0


def test_no_edges_at_all(cuda):
    pos = np.array([[1.0, 1.0, 1.0], [50.0, 50.0, 50.0]], np.float32)
    ei, cs, g = _check_vs_oracle(pos, (np.eye(3) * 100).astype(np.float32), [True, True, True], 3.0, cuda, what="sparse")
    assert g["E"] == 0


def test_target_subset_unsorted_with_duplicates(cuda):
    pos, cell, pbc = _cubic(800, 25.0, 21)
    rng = np.random.default_rng(5)
    targets = rng.permutation(800)[:300].astype(np.int64)
    targets[10] = targets[3]  # a duplicate entry is a separate target
    _check_vs_oracle(pos, cell, pbc, 5.0, cuda, targets=targets, what="subset")


@pytest.mark.parametrize("case", ["x", "xyz", "thin_gap", "pbc_xy", "triclinic", "unwrapped"])
def test_target_subset_touching_the_periodic_boundary(cuda, case):
    """A rank's atoms form a compact subdomain that wraps around the periodic boundary: after the wrap the
    targets sit at both ends of the box and the grid spans it, with the cell scan walking only the groups that hold
    targets; the edges must be the oracle's in every case."""
    rng = np.random.default_rng(606)
    n, L, r = 20000, 80.0, 5.0
    cell = (np.eye(3) * L).astype(np.float32)
    pbc = [True, True, True]
    pos = (rng.random((n, 3)) * L).astype(np.float32)

    def arc(c, lo, hi):     # coordinates in [lo, L) or [0, hi)
        return (c >= lo) | (c < hi)

    if case == "x":
        sel = arc(pos[:, 0], 70.0, 18.0)
    elif case == "xyz":
        sel = arc(pos[:, 0], 66.0, 12.0) & arc(pos[:, 1], 75.0, 20.0) & arc(pos[:, 2], 60.0, 5.0)
    elif case == "thin_gap":   # the empty stretch is shorter than twice the reach: no shifted frame, still right
        sel = arc(pos[:, 0], 12.0, 4.0)
    elif case == "pbc_xy":
        pbc = [True, True, False]
        sel = arc(pos[:, 0], 70.0, 18.0) & arc(pos[:, 2], 0.0, 30.0)
    elif case == "triclinic":
        cell = np.array([[L, 0, 0], [0.2 * L, L, 0], [0.1 * L, 0, L]], dtype=np.float32)
        pos = (rng.random((n, 3)) @ cell.astype(np.float64)).astype(np.float32)
        sel = arc(pos[:, 0], 70.0, 18.0)
    else:                      # targets given outside the cell: x in [-10, 18) wraps to [70, 80) and [0, 18)
        pos[:, 0] = pos[:, 0] - 10.0
        sel = pos[:, 0] < 18.0
    targets = np.nonzero(sel)[0].astype(np.int64)
    assert 100 < targets.size < n
    _check_vs_oracle(pos, cell, pbc, r, cuda, targets=targets, what=case)
    # the owned atoms first, as a rank holds them ([owned | halo] with targets 0..n_own-1)
    order = np.concatenate([targets, np.nonzero(~sel)[0]])
    _check_vs_oracle(pos[order], cell, pbc, r, cuda, targets=np.arange(targets.size, dtype=np.int64), what=case + "/owned first")


def test_counts_only_matches(cuda):
    import dynamis_b200 as D

    pos, cell, pbc = _cubic(600, 22.0, 31)
    targets = np.arange(0, 600, 3, dtype=np.int64)
    c = D.radius_graph_pbc_counts_ex(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc),
                                     5.0, torch.as_tensor(targets, device=cuda))
    g = O.radius_graph(pos, cell, pbc, 5.0, targets)
    np.testing.assert_array_equal(c.cpu().numpy(), g["counts"])


def test_bad_target_raises(cuda):
    import dynamis_b200 as D

    pos, cell, pbc = _cubic(50, 10.0, 2)
    with pytest.raises(RuntimeError, match="outside"):
        D.radius_graph_pbc_ex(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), 3.0, 0, False,
                              torch.tensor([0, 50], device=cuda))


def test_validation_messages(cuda):
    import dynamis_b200 as D

    pbc = torch.tensor([True, True, True])
    with pytest.raises(RuntimeError, match="pos must be a CUDA tensor"):
        D.radius_graph_pbc(torch.zeros(4, 3), torch.eye(3), pbc, 1.0, 0, False)
    with pytest.raises(RuntimeError, match=r"pos must have shape \[N, 3\]"):
        D.radius_graph_pbc(torch.zeros(4, 2, device=cuda), torch.eye(3), pbc, 1.0, 0, False)
    with pytest.raises(RuntimeError, match="radius must be positive"):
        D.radius_graph_pbc(torch.zeros(4, 3, device=cuda), torch.eye(3), pbc, 0.0, 0, False)
    with pytest.raises(RuntimeError, match="target_indices must be int64"):
        D.radius_graph_pbc_ex(torch.zeros(4, 3, device=cuda), torch.eye(3), pbc, 1.0, 0, False,
                              torch.zeros(2, dtype=torch.int32, device=cuda))


def test_wrapper_batch(cuda):
    import dynamis_b200 as D

    class Data:
        pass

    rng = np.random.default_rng(9)
    d = Data()
    d.pos = torch.as_tensor((rng.random((90, 3)) * 12.0).astype(np.float32), device=cuda)
    d.cell = (torch.eye(3, device=cuda) * 12.0).unsqueeze(0).repeat(2, 1, 1)
    d.natoms = torch.tensor([40, 50], device=cuda)
    d.pbc = torch.tensor([[True, True, True], [True, True, True]])
    ei, co, nn = D.radius_graph_pbc_cuda(d, 4.0, 100)
    assert nn.shape == (2,) and int(nn.sum()) == ei.size(1)
    p = d.pos.cpu().numpy()
    cell = (np.eye(3) * 12.0).astype(np.float32)
    g0 = O.radius_graph(p[:40], cell, [1, 1, 1], 4.0)
    g1 = O.radius_graph(p[40:], cell, [1, 1, 1], 4.0)
    ref = O.canonical_edges(np.concatenate([g0["src"], g1["src"] + 40]), np.concatenate([g0["dst"], g1["dst"] + 40]),
                            np.concatenate([g0["shift"], g1["shift"]]))
    assert_same_edges(canon_t(ei, co), ref, "batch wrapper")


def test_cutoff_tie_stress(cuda):
    """Pairs placed within a few ulp of the cutoff: membership hinges on the exact fp32 rounding of
    d2 = dx*dx + dy*dy + dz*dz, so the kernel and the oracle must round identically."""
    rng = np.random.default_rng(77)
    n_pairs = 4000
    box = 400.0
    r = np.float32(5.0)
    base = (rng.random((n_pairs, 3)) * (box - 20) + 10).astype(np.float32)
    dirs = rng.normal(size=(n_pairs, 3))
    dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
    other = np.empty_like(base)
    for i in range(n_pairs):
        p = (base[i].astype(np.float64) + dirs[i] * float(r)).astype(np.float32)
        ax = int(rng.integers(0, 3))
        for _ in range(int(rng.integers(0, 5))):
            p[ax] = np.nextafter(p[ax], np.float32(np.inf if rng.random() < 0.5 else -np.inf), dtype=np.float32)
        other[i] = p
    pos = np.concatenate([base, other]).astype(np.float32)
    ei, cs, g = _check_vs_oracle(pos, (np.eye(3) * box).astype(np.float32), [True, True, True], float(r), cuda, what="ties")
    # the construction must actually straddle the cutoff
    assert 0.15 * 2 * n_pairs < g["E"] < 0.85 * 2 * n_pairs + 50000


def test_config1_fcc_32k(cuda):
    pos, cell, pbc, r = synthetic.fcc_copper(20)
    ei, cs, g = _check_vs_oracle(pos, cell, pbc, r, cuda, what="fcc 32k")
    assert g["E"] == 2485474


def test_float64_triclinic_small(cuda):
    pos, cell, pbc, r = synthetic.triclinic_silicon(6, 6, 3)
    assert pos.dtype == np.float64
    import dynamis_b200 as D

    out = D.radius_graph_pbc_with_dist(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), r)
    ei, cs, nni, counts, d2 = out
    g = O.radius_graph(pos, cell, pbc, r)
    assert_same_edges(canon_t(ei, cs), canon_o(g), "fp64 triclinic")
    # distances: recompute in float64 from the returned edges; tolerance 1e-12 relative
    p = torch.as_tensor(pos, device=cuda)
    c = torch.as_tensor(cell, device=cuda)
    vec = p[ei[0]] + cs.double() @ c - p[ei[1]]
    torch.testing.assert_close(d2, (vec * vec).sum(dim=1), rtol=1e-12, atol=1e-12)


def test_edge_distances_fp32(cuda):
    import dynamis_b200 as D

    pos, cell, pbc = _cubic(2000, 35.0, 55)
    out = D.radius_graph_pbc_with_dist(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), 5.0)
    ei, cs, nni, counts, d2 = out
    g = O.radius_graph(pos, cell, pbc, 5.0)
    # same edges -> compare d2 edge by edge after canonical ordering
    ours = canon_t(ei, cs)
    order_o = np.lexsort((g["shift"][:, 2], g["shift"][:, 1], g["shift"][:, 0], g["src"], g["dst"]))
    ein = ei.cpu().numpy()
    csn = np.rint(cs.cpu().numpy()).astype(np.int64)
    order_t = np.lexsort((csn[:, 2], csn[:, 1], csn[:, 0], ein[0], ein[1]))
    assert_same_edges(ours, canon_o(g), "dist edges")
    np.testing.assert_allclose(d2.cpu().numpy()[order_t], g["d2"][order_o], rtol=1e-6)


@pytest.mark.parametrize("periodic", [True, False])
def test_image_capacity_overflow_is_reported_and_the_plan_repeated(cuda, periodic):
    """A capacity for the periodic images that turns out too small must come back as a status bit with the true
    count (so that the caller can repeat the plan), not as a write past the buffers: on the fully periodic path the
    scatter pass is the first to know, otherwise the grid kernel.  The host layer's capacity cache is made too
    small on purpose; the call must still return the right graph."""
    from dynamis_b200 import graph as G

    pos, cell, pbc = _cubic(4000, 30.0, 5)
    if not periodic:
        pbc = [True, True, False]
    geo = G._dev_state(cuda)["geo"]
    geo.clear()
    try:
        _check_vs_oracle(pos, cell, pbc, 5.0, cuda, what="first call")
        assert len(geo) == 1, "the first call should have left its capacities in the cache"
        (key, (cell_h, pbc_h, radius, src_cap, cell_cap)), = geo.items()
        geo[key] = (cell_h, pbc_h, radius, 1000, cell_cap)      # fewer slots than atoms, let alone images
        _check_vs_oracle(pos, cell, pbc, 5.0, cuda, what="after the overflow")
        assert geo[key][3] > 4000, "the repeated plan should have left the larger capacity in the cache"
    finally:
        geo.clear()


# ------------------------------------------------------------------ against the reference's own kernels

def _run_ref(ref_ops, pos, cell, pbc, r, dev, targets=None):
    tp = torch.as_tensor(pos, device=dev)
    tc = torch.as_tensor(cell, device=dev)
    tb = torch.as_tensor(np.asarray(pbc, dtype=bool), device=dev)
    tt = torch.as_tensor(targets, device=dev) if targets is not None else None
    return ref_ops.radius_graph(tp, tc, tb, float(r), tt, False)


@pytest.mark.parametrize("case", ["cubic1000", "multi_image", "triclinic", "pbc_xy", "no_pbc", "unwrapped", "subset", "fcc32k"])
def test_vs_reference_kernels(cuda, ref_ops, case):
    targets = None
    if case == "cubic1000":
        pos, cell, pbc = _cubic(1000, 30.0, 2024); r = 5.0
    elif case == "multi_image":
        pos, cell, pbc = _cubic(30, 8.0, 7); r = 6.0
    elif case == "triclinic":
        rng = np.random.default_rng(3)
        cell = np.array([[12.0, 0.0, 0.0], [2.5, 11.0, 0.0], [1.5, -2.0, 13.0]], np.float32)
        pos = (rng.random((400, 3)) @ cell.astype(np.float64)).astype(np.float32); pbc = [True] * 3; r = 5.0
    elif case == "pbc_xy":
        pos, cell, _ = _cubic(300, 14.0, 11); pbc = [True, True, False]; r = 4.5
    elif case == "no_pbc":
        pos, cell, _ = _cubic(300, 14.0, 12); pbc = [False] * 3; r = 4.5
    elif case == "unwrapped":
        rng = np.random.default_rng(14)
        pos = ((rng.random((500, 3)) - 0.5) * 60.0).astype(np.float32); cell = (np.eye(3) * 15.0).astype(np.float32)
        pbc = [True] * 3; r = 4.0
    elif case == "subset":
        pos, cell, pbc = _cubic(800, 25.0, 21); r = 5.0
        targets = np.random.default_rng(5).permutation(800)[:300].astype(np.int64)
    else:
        pos, cell, pbc, r = synthetic.fcc_copper(20)
    ei, cs, nni, counts = _run_ours(pos, cell, pbc, r, cuda, targets)
    rei, rcs, rnn, rcounts = _run_ref(ref_ops, pos, cell, pbc, r, cuda, targets)
    assert_same_edges(canon_t(ei, cs), canon_t(rei, rcs), f"vs reference: {case}")
    assert torch.equal(counts, rcounts)
    assert int(nni.item()) == int(rnn.item())


def test_vs_reference_kernels_1m_digest(cuda, ref_ops):
    """The single-GPU benchmark workload (1,000,000 random atoms, r = 5): count and an order-independent
    64-bit digest of the edge set must equal the reference's."""
    pos, cell, pbc, r = synthetic.random_liquid(1_000_000)
    ei, cs, nni, counts = _run_ours(pos, cell, pbc, r, cuda)
    mine = digest_t(ei, cs)
    cnt_sum = int(counts.sum().item())
    del ei, cs
    rei, rcs, rnn, rcounts = _run_ref(ref_ops, pos, cell, pbc, r, cuda)
    theirs = digest_t(rei, rcs)
    assert mine == theirs
    assert cnt_sum == mine[0]
    assert torch.equal(counts, rcounts)
