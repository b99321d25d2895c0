"""Model-side graph glue written by the edge writer (reference: dynamis_model/src/dynamis_model/nnp/mace.py:591-608
`_radius_graph` / `_build_owned_graph`, uma.py:915-948).

The reference composition is restated with torch on the full graph: negate the offsets, keep the edges
whose destination is owned, multiply by the cell.  `owned_graph` must give the same edge set with the
same unit shifts, and Cartesian shifts equal to torch.matmul's (bit-exact expected: K = 3 float32 GEMM;
the test accepts 1e-6 relative as the stated fp32 tolerance and reports exactness separately).
"""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from dynamis_b200 import synthetic

pytestmark = pytest.mark.gpu


def _canon(ei, unit, extra=None):
    """Sort edges by (dst, src, shift) and return the arrays in that order."""
    u = unit.round().to(torch.int64) + 512
    key2 = (u[:, 0] << 20) | (u[:, 1] << 10) | u[:, 2]
    order = torch.argsort(key2, stable=True)
    order = order[torch.argsort(ei[0][order], stable=True)]
    order = order[torch.argsort(ei[1][order], stable=True)]
    out = [ei[:, order], unit[order]]
    if extra is not None:
        out.append(extra[order])
    return out


def _reference_composition(pos, cell, pbc, cutoff, num_local):
    ei, off, _, _ = D.radius_graph_pbc_ex(pos, cell, pbc, cutoff, 0, False)
    unit = -off                                       # mace.py:598
    keep = ei[1] < num_local                          # mace.py:605
    ei = ei[:, keep].contiguous()
    unit = unit[keep].to(torch.float32)
    shifts = torch.matmul(unit, cell.to(pos.device).reshape(3, 3).to(torch.float32))  # mace.py:609
    return ei, unit, shifts


CASES = {
    "triclinic": lambda: synthetic.triclinic_silicon(6, 6, 4),
    "liquid": lambda: synthetic.random_liquid(20_000, seed=5),
    "fcc_thin_slab": lambda: synthetic.fcc_copper(6, seed=3),
}


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("frac_local", [1.0, 0.6, 0.02])
def test_owned_graph_equals_reference_composition(cuda, name, frac_local):
    pos, cell, pbc, r = CASES[name]()
    pos = pos.astype(np.float32)
    n = pos.shape[0]
    num_local = max(1, int(n * frac_local))
    tp = torch.as_tensor(pos, device=cuda)
    tc = torch.as_tensor(cell.astype(np.float32))
    tb = torch.tensor(pbc)
    ei, unit, cart = D.owned_graph(tp, tc, tb, r, num_local)
    rei, runit, rcart = _reference_composition(tp, tc, tb, r, num_local)
    assert ei.shape == rei.shape and int(ei[1].max()) < num_local
    a = _canon(ei, unit, cart)
    b = _canon(rei, runit, rcart)
    assert torch.equal(a[0], b[0])
    assert torch.equal(a[1], b[1])
    torch.testing.assert_close(a[2], b[2], rtol=1e-6, atol=1e-6)
    exact = bool(torch.equal(a[2], b[2]))
    print(f"{name} frac_local={frac_local}: E={ei.shape[1]}, Cartesian shifts bit-exact vs torch.matmul: {exact}")


def test_owned_graph_signs_and_optional_outputs(cuda):
    pos, cell, pbc, r = synthetic.random_liquid(5_000, seed=11)
    tp = torch.as_tensor(pos.astype(np.float32), device=cuda)
    tc, tb = torch.as_tensor(cell.astype(np.float32)), torch.tensor(pbc)
    ei_n, unit_n, cart_n = D.owned_graph(tp, tc, tb, r, 3000, negate_shifts=True)
    ei_p, unit_p, none = D.owned_graph(tp, tc, tb, r, 3000, negate_shifts=False, cartesian=False)
    assert none is None
    assert torch.equal(ei_n, ei_p)                 # same plan, same edge order
    assert torch.equal(unit_n, -unit_p)
    # the un-negated shifts are those of radius_graph_pbc_ex on the same target subset
    e2, s2, _, _ = D.radius_graph_pbc_ex(tp, tc, tb, r, 0, False, torch.arange(3000, device=cuda))
    assert torch.equal(e2, ei_p) and torch.equal(s2, unit_p)
    assert bool((unit_n != 0).any())               # the box is periodic: some edges cross it
    # ids written through a map (local -> global, as DistGraphBuilder's steady build needs them)
    from dynamis_b200.graph import plan_radius_graph
    gid = torch.randperm(5_000, device=cuda) + 1_000_000
    plan = plan_radius_graph(tp, tc, tb, r, torch.arange(3000, device=cuda))
    e_map, s_map, _ = plan.fill_glue(None, negate_shifts=False, cartesian=False, id_map=gid)
    assert torch.equal(e_map, gid[ei_p]) and torch.equal(s_map, unit_p)


def test_owned_graph_degenerate(cuda):
    pos, cell, pbc, r = synthetic.random_liquid(2_000, seed=2)
    tp = torch.as_tensor(pos.astype(np.float32), device=cuda)
    tc, tb = torch.as_tensor(cell.astype(np.float32)), torch.tensor(pbc)
    ei, unit, cart = D.owned_graph(tp, tc, tb, r, 0)
    assert ei.shape == (2, 0) and unit.shape == (0, 3) and cart.shape == (0, 3)
    with pytest.raises(RuntimeError):
        D.owned_graph(tp, tc, tb, r, 2_001)
    from dynamis_b200 import _lib

    lib = _lib.lib()
    assert lib.dynb_rg_fill_glue(None, 0, None, None, None, None, 1, None, 5, None) != 0
    assert b"workspace" in lib.dynb_last_error()
