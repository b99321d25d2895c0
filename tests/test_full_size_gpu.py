"""Full-size parity and property tests on one B200 (the sizes of the benchmark configurations).

  * 1,000,000-atom liquid (fp32) and 500,000-atom triclinic Si (fp64): count and order-independent
    64-bit digest of the edge set equal the CPU oracle's.
  * 8,001,504-atom fcc Cu (fp32, 613 M edges): size-independent properties — degrees sum to E, every
    edge vector recomputed from (src, dst, shift) is inside the cutoff and not a self pair, edge ids are
    in range, and the number of directed edges whose reverse is missing is negligible (only pairs within
    an ulp of the cutoff may be one-directional, because image positions round differently per direction).
"""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from _util import digest_t
from dynamis_b200 import synthetic
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def test_liquid_1m_digest_vs_oracle(cuda):
    pos, cell, pbc, r = synthetic.random_liquid(1_000_000)
    ei, cs, nni, counts = D.radius_graph_pbc_ex(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), r, 0, False)
    g = O.radius_graph(pos, cell, pbc, r)
    assert digest_t(ei, cs) == O.edge_set_digest(g["src"], g["dst"], g["shift"])
    np.testing.assert_array_equal(counts.cpu().numpy(), g["counts"])


def test_triclinic_si_500k_fp64_digest_vs_oracle(cuda):
    pos, cell, pbc, r = synthetic.triclinic_silicon()
    assert pos.shape == (500_000, 3) and pos.dtype == np.float64
    ei, cs, nni, counts, d2 = D.radius_graph_pbc_with_dist(torch.as_tensor(pos, device=cuda), torch.as_tensor(cell), torch.tensor(pbc), r)
    g = O.radius_graph(pos, cell, pbc, r)
    assert digest_t(ei, cs) == O.edge_set_digest(g["src"], g["dst"], g["shift"])
    np.testing.assert_array_equal(counts.cpu().numpy(), g["counts"])
    # fp64 distances, 1e-12 relative, on a slice (edge order differs from the oracle's: recompute instead)
    p, c = torch.as_tensor(pos, device=cuda), torch.as_tensor(cell, device=cuda)
    sl = slice(0, 2_000_000)
    vec = p[ei[0, sl]] + cs[sl].double() @ c - p[ei[1, sl]]
    torch.testing.assert_close(d2[sl], (vec * vec).sum(dim=1), rtol=1e-12, atol=1e-12)


def test_fcc_8m_properties(cuda):
    free, _ = torch.cuda.mem_get_info(cuda)
    if free < 70 * (1 << 30):
        pytest.skip("needs about 60 GB of free device memory")
    pos, cell, pbc, r = synthetic.fcc_copper(126, seed=1004)
    assert pos.shape[0] == 8_001_504
    p = torch.as_tensor(pos, device=cuda)
    c = torch.as_tensor(cell, device=cuda)
    ei, cs, nni, counts = D.radius_graph_pbc_ex(p, torch.as_tensor(cell), torch.tensor(pbc), r, 0, False)
    E = int(nni.item())
    assert ei.shape == (2, E) and int(counts.sum(dtype=torch.int64).item()) == E
    assert 75.0 < E / pos.shape[0] < 79.0
    assert int(ei.min()) >= 0 and int(ei.max()) < pos.shape[0]
    assert torch.equal(torch.bincount(ei[1], minlength=pos.shape[0]).to(torch.int32), counts)
    # every edge vector is inside the cutoff and not a self pair (checked in chunks, in float64)
    pd, cd = p.double(), c.double()
    step = 40_000_000
    for a in range(0, E, step):
        s = slice(a, min(E, a + step))
        vec = pd[ei[0, s]] + cs[s].double() @ cd - pd[ei[1, s]]
        d2 = (vec * vec).sum(dim=1)
        assert float(d2.max()) <= r * r * (1 + 1e-5) and float(d2.min()) > 1e-8
        del vec, d2
    # symmetry: sum of per-edge hashes of (src, dst, shift) vs (dst, src, -shift)
    fwd = digest_t(ei, cs)
    rev = digest_t(torch.stack([ei[1], ei[0]]), -cs)
    if fwd != rev:
        # count one-directional edges exactly via sorted 64-bit keys (rare path)
        def keys(e0, e1, sh):
            s = sh.round().to(torch.int64) + 4
            return (e0 << 40) ^ (e1 << 12) ^ (s[:, 0] << 8) ^ (s[:, 1] << 4) ^ s[:, 2]
        kf = torch.sort(keys(ei[0], ei[1], cs)).values
        kr = torch.sort(keys(ei[1], ei[0], -cs)).values
        idx = torch.searchsorted(kr, kf).clamp_(max=kr.numel() - 1)
        missing = int((kr[idx] != kf).sum())
        assert missing <= 64, f"{missing} directed edges have no reverse edge"
