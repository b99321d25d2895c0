"""CPU tests of the boundary: the C-ABI library loads and exports every symbol include/dynb.h
declares, argument validation that needs no GPU, host-side logic, and the N > 1 exchange plan over a
world_size-2 gloo group."""

import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from dynamis_b200 import _lib

    L = _lib.lib()
    header = open(os.path.join(ROOT, "include", "dynb.h")).read()
    declared = set(re.findall(r"\b(dynb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in dynb.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert L.dynb_version() >= 1


def test_argument_validation_without_gpu():
    from dynamis_b200 import _lib

    L = _lib.lib()
    n = ctypes.c_int64()
    assert L.dynb_rg_workspace_bytes(-1, 1, 1, 1, 0, ctypes.byref(n)) == -1
    assert b"bad arguments" in L.dynb_last_error()
    assert L.dynb_rg_workspace_bytes(1000, 1000, 2000, 5000, 0, ctypes.byref(n)) == 0 and n.value > 0
    f32 = n.value
    assert L.dynb_rg_workspace_bytes(1000, 1000, 2000, 5000, 1, ctypes.byref(n)) == 0 and n.value > f32
    cell = np.eye(3, dtype=np.float32) * 20
    pbc = np.ones(3, np.uint8)
    a, b = ctypes.c_int64(), ctypes.c_int64()
    assert L.dynb_rg_suggest_capacity(1000, cell.ctypes.data, pbc.ctypes.data, 5.0, 0, ctypes.byref(a), ctypes.byref(b)) == 0
    assert 1000 <= a.value <= 27000 and b.value >= 8 ** 3
    assert L.dynb_rg_suggest_capacity(1000, cell.ctypes.data, pbc.ctypes.data, -1.0, 0, ctypes.byref(a), ctypes.byref(b)) == -1
    sing = np.zeros((3, 3), np.float32)
    assert L.dynb_rg_suggest_capacity(10, sing.ctypes.data, pbc.ctypes.data, 5.0, 0, ctypes.byref(a), ctypes.byref(b)) == -1
    assert L.dynb_sfc_workspace_bytes(1000, ctypes.byref(n)) == 0 and n.value > 0
    assert L.dynb_sfc_partition(None, 10, None, 0, 0, None, None, None, 0, None) == -1  # W < 1
    assert L.dynb_radix_sort_pairs(None, None, 10, 3, 64, None, 0, None) == -1  # begin_bit not a multiple of 8


def test_host_geometry_matches_oracle_restatement():
    """dynb_rg_suggest_capacity runs the library's host cell geometry; its image-capacity bound must
    be consistent with the oracle's replication counts (reference: radius_graph_kernels.cu:516-571)."""
    from dynamis_b200 import _lib
    from oracle import cpu_oracle as O

    L = _lib.lib()
    for cell, r in ((np.eye(3) * 5.0, 6.0), (np.eye(3) * 72.3, 6.0), (np.array([[12.0, 0, 0], [2.5, 11, 0], [1.5, -2, 13]]), 5.0)):
        cell = cell.astype(np.float32)
        rep, cf, inv = O.geometry(cell, [1, 1, 1], r)
        np.testing.assert_allclose(inv @ cell, np.eye(3), atol=1e-5)
        a, b = ctypes.c_int64(), ctypes.c_int64()
        pbc = np.ones(3, np.uint8)
        assert L.dynb_rg_suggest_capacity(100, cell.ctypes.data, pbc.ctypes.data, r, 0, ctypes.byref(a), ctypes.byref(b)) == 0
        assert a.value <= 100 * int(np.prod(2 * rep + 1))
        assert a.value >= 100


def test_python_validation_messages_without_gpu():
    import dynamis_b200 as D

    pbc = torch.tensor([True, True, True])
    with pytest.raises(RuntimeError, match="pos must be a CUDA tensor"):
        D.radius_graph_pbc(torch.zeros(4, 3), torch.eye(3), pbc, 1.0, 0, False)
    with pytest.raises(RuntimeError, match="pos must be a CUDA tensor"):
        D.sfc_partition_labels(torch.zeros(4, 3), None, 2, 0)
    with pytest.raises(RuntimeError, match="edges must be a CUDA tensor"):
        D.filter_edges_to_radius(torch.zeros(2, 0, dtype=torch.int64), torch.zeros(0, 3), torch.zeros(4, 3), torch.eye(3), 1.0)
    with pytest.raises(RuntimeError, match="input must be a CUDA tensor"):
        D.push_buffer_create(torch.zeros(2, 2), torch.zeros(1, 2), torch.zeros(1, dtype=torch.int64))
    info = D.PartitionMessagePassingInfo()
    assert info.send_offsets is None and info.edge_index_halo is None  # unset tensor fields read back as None
    info._edge_index_halo_fn = lambda: torch.zeros(2, 3, dtype=torch.int64)
    assert info.edge_index_halo.shape == (2, 3)
    st = D.DynamisState()
    st.dist_env.world_size = 8
    assert st.dist_env.world_size == 8 and st.local_partition_info.partition_id is None
    assert int(D.SFCCurveType.Morton) == 0 and int(D.SFCCurveType.Hilbert) == 1


def test_synthetic_configs_have_the_stated_shapes():
    from dynamis_b200 import synthetic as S

    pos, cell, pbc, r = S.fcc_copper(20)
    assert pos.shape == (32000, 3) and pos.dtype == np.float32 and abs(cell[0, 0] - 72.3) < 1e-4 and r == 6.0
    pos, cell, pbc, r = S.random_liquid(1000)
    assert abs(cell[0, 0] - (1000 / 0.1) ** (1 / 3)) < 1e-3 and r == 5.0
    assert abs((1_000_000 / 0.1) ** (1 / 3) - 215.44) < 0.01
    pos, cell, pbc, r = S.triclinic_silicon(2, 2, 1)
    assert pos.shape == (32, 3) and pos.dtype == np.float64 and cell[1, 0] > 0 and cell[2, 0] > 0 and cell[2, 1] == 0
    assert 126 ** 3 * 4 == 8_001_504


WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import cpu_oracle as O
from dynamis_b200.exchange import _PlanCache
from dynamis_b200.state import PartitionMessagePassingInfo
rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
rng = np.random.default_rng(5)
pos = (rng.random((1500, 3)) * 30).astype(np.float32); cell = (np.eye(3) * 30).astype(np.float32)
g = O.radius_graph(pos, cell, [1, 1, 1], 5.5)
pid = O.sfc_partition(pos, None, W, 0)
maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
m = maps[rank]
info = PartitionMessagePassingInfo()
info.send_offsets = torch.as_tensor(m["send_offsets"]); info.recv_offsets = torch.as_tensor(m["recv_offsets"])
info.send_local_indices = torch.as_tensor(m["send_local_indices"])
# host logic under test: the cached split lists of the exchanger (no device work)
c = _PlanCache.__new__(_PlanCache); c.key = None
so, ro = info.send_offsets.tolist(), info.recv_offsets.tolist()
send_splits = [so[r + 1] - so[r] for r in range(W)]; recv_splits = [ro[r + 1] - ro[r] for r in range(W)]
# every rank's recv split from a peer must equal that peer's send split to it
all_send = [None] * W
dist.all_gather_object(all_send, send_splits)
assert [all_send[p][rank] for p in range(W)] == recv_splits
F = 4
feats = [np.arange(mm["num_local"] * F, dtype=np.float32).reshape(-1, F) + 1000 * r for r, mm in enumerate(maps)]
x = torch.as_tensor(feats[rank])
send = x[info.send_local_indices]
out = torch.empty((m["num_local"] + ro[-1], F))
out[:m["num_local"]] = x
recv_chunks = [torch.empty((n, F)) for n in recv_splits]
reqs = []
for p, chunk in enumerate(torch.split(send, send_splits)):
    if p != rank and chunk.numel():
        reqs.append(dist.isend(chunk.contiguous(), p))
for p in range(W):
    if p != rank and recv_chunks[p].numel():
        reqs.append(dist.irecv(recv_chunks[p], p))
for q in reqs:
    q.wait()
out[m["num_local"]:] = torch.cat(recv_chunks)
ref = O.exchange_forward(feats, [mm["send_offsets"] for mm in maps], [mm["send_local_indices"] for mm in maps], [mm["recv_offsets"] for mm in maps])
assert np.array_equal(out.numpy(), ref[rank])
dist.barrier(); dist.destroy_process_group()
'''


def test_exchange_plan_over_gloo_world_size_2(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
