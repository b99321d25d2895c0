"""Worker for test_multi_gpu.py: one rank per GPU under torchrun.  Builds a halo plan for a small
system (CPU oracle), runs both exchangers forward and backward on real GPUs and checks the results
against the oracle.  Exits non-zero on any mismatch."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import dynamis_b200 as D  # noqa: E402
from oracle import cpu_oracle as O  # noqa: E402


def main():
    rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    rng = np.random.default_rng(99)
    n, L = 20000, 64.0
    pos = (rng.random((n, 3)) * L).astype(np.float32)
    cell = (np.eye(3) * L).astype(np.float32)

    # partition + halo maps through the product path on this rank's GPU
    st = D.MolecularInfo()
    st.num_atoms, st.atom_positions = n, torch.as_tensor(pos, device=dev)
    st.atom_vertex_numbers = torch.arange(n, dtype=torch.int64, device=dev)
    env = D.DistEnvironment()
    env.global_rank, env.world_size = rank, W
    cfg = D.SimulationConfig()
    cfg.cutoff, cfg.ghost_cutoff_buffer, cfg.cell, cfg.pbc = 6.0, 0.5, torch.as_tensor(cell), torch.tensor([True] * 3)
    part = D.SFCPartitioner()
    info = part.partition(st, env)
    part.build_halo_maps(info, st, env, cfg)

    # the oracle's view of every rank
    g = O.radius_graph(pos, cell, [1, 1, 1], np.float32(6.5))
    pid = O.sfc_partition(pos, None, W, 0)
    maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
    assert np.array_equal(info.send_local_indices.cpu().numpy(), maps[rank]["send_local_indices"])
    assert np.array_equal(info.recv_offsets.cpu().numpy(), maps[rank]["recv_offsets"])
    so = [m["send_offsets"] for m in maps]
    sl = [m["send_local_indices"] for m in maps]
    ro = [m["recv_offsets"] for m in maps]
    nl = [m["num_local"] for m in maps]
    state = D.DynamisState()
    state.local_partition_info = info

    for make in (lambda: D.GPUDirectExchanger(wait_ns=10_000_000_000), lambda: D.PythonNCCLExchanger()):
        for F in (3, 128):
            ex = make()
            frng = np.random.default_rng(1234 + F)
            feats = [frng.standard_normal((nl[r], F)).astype(np.float32) for r in range(W)]
            ref = O.exchange_forward(feats, so, sl, ro)
            grads = [frng.standard_normal(ref[r].shape).astype(np.float32) for r in range(W)]
            refb = O.exchange_backward(grads, nl, so, sl, ro)
            for it in range(3):
                x = torch.as_tensor(feats[rank], device=dev).requires_grad_(True)
                out = D.FeaturePushToExchange.apply(x, state, ex)
                assert np.array_equal(out.detach().cpu().numpy(), ref[rank]), f"forward mismatch {type(ex).__name__} F={F}"
                out.backward(torch.as_tensor(grads[rank], device=dev))
                np.testing.assert_allclose(x.grad.cpu().numpy(), refb[rank], rtol=1e-6, atol=1e-6)
            if hasattr(ex, "exchanger"):
                ex.exchanger.check_status()
            dist.barrier()
            ex.reset_buffers()
    # the drift word rides on the handshake of every push (reference: comm/drift_flags.py,
    # dynamis/tests/test_drift_watchdog.py:97-120): one rank raises a bit, every rank sees it after the push
    flags = D.drift_flags.enable(dev)
    ex = D.GPUDirectExchanger(wait_ns=10_000_000_000)
    F = 8
    x = torch.randn(nl[rank], F, device=dev)
    for it in range(8):
        word = (1 + (it % 3)) if (it % W == rank and it % 2 == 0) else 0
        flags.local.fill_(word)
        out = ex.feature_push_forward(x, info)
        assert int(flags.global_.item()) == ((1 + (it % 3)) if it % 2 == 0 else 0), f"drift word, generation {it}"
        flags.local.fill_(2 if rank == W - 1 else 0)
        ex.feature_push_backward(torch.ones_like(out), x.shape, info)
        assert int(flags.global_.item()) == 2
    assert flags.n_wired == 1
    D.drift_flags.disable(dev)
    dist.barrier()
    ex.reset_buffers()

    # the reference's own set-up sequence (comm/exchanger.py:401-536): caller-allocated buffers, handles
    # gathered over the process group, setup_ipc with 13 arguments, sync handle, setup_sync
    def gather_bytes(h):
        lst = [None] * W
        dist.all_gather_object(lst, list(h))
        return lst

    total_recv, total_send = int(info.recv_offsets[-1]), int(info.send_offsets[-1])
    all_ro = [torch.zeros(W + 1, dtype=torch.int64, device=dev) for _ in range(W)]
    dist.all_gather(all_ro, info.recv_offsets.to(dev))
    all_ro = torch.stack(all_ro)
    all_nl = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(W)]
    dist.all_gather(all_nl, torch.tensor([nl[rank]], dtype=torch.int64, device=dev))
    all_nl = torch.cat(all_nl)
    frng = np.random.default_rng(4321)
    feats = [frng.standard_normal((nl[r], F)).astype(np.float32) for r in range(W)]
    ref = O.exchange_forward(feats, so, sl, ro)
    grads = [frng.standard_normal(ref[r].shape).astype(np.float32) for r in range(W)]
    refb = O.exchange_backward(grads, nl, so, sl, ro)
    for cls in (D.FeatureExchanger, D.IPCExchanger):
        e = cls(wait_ns=10_000_000_000)
        xb = cls.allocate_ipc_buffer(max(1, nl[rank] + total_recv), F, dev.index)
        gb = cls.allocate_ipc_buffer(max(1, total_send), F, dev.index)
        assert xb.shape == (max(1, nl[rank] + total_recv), F) and xb.is_cuda and float(xb.abs().sum()) == 0.0
        hx, hg = e.export_ipc_handle(xb), e.export_ipc_handle(gb)
        assert len(hx) == 64 and all(isinstance(v, int) for v in hx)
        args = (xb, gb, gather_bytes(hx), gather_bytes(hg), info.send_offsets, info.send_local_indices.to(dev),
                info.recv_offsets, all_ro, all_nl, nl[rank], F, rank, W)
        if cls is D.FeatureExchanger:
            e.setup_ipc(*args)
        else:
            e.setup(*args)
        e.setup_sync(gather_bytes(e.create_and_export_sync_handle()))
        word, seen = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
        e.set_watchdog_flags(word, seen)
        word.fill_(4 if rank == 0 else 0)
        xt, gt = torch.as_tensor(feats[rank], device=dev), torch.as_tensor(grads[rank], device=dev)
        for it in range(3):
            if cls is D.FeatureExchanger:
                assert e.is_ipc_setup()
                out = e.feature_push_forward(xt, info)
                back = e.feature_push_backward(gt, xt.shape, info)
            else:
                assert e.is_setup() and not e.use_fabric()
                xb[:nl[rank]].copy_(xt)
                e.push_forward(xb)
                e.record_push_complete()
                e.wait_for_pushes()
                out = xb.clone()
                dist.barrier()          # caller-owned single buffers: nobody may push again before all have read
                e.push_backward(gt)
                e.record_push_complete()
                e.wait_for_pushes()
                back = gt[:nl[rank]].clone().index_add_(0, info.send_local_indices.to(dev), gb[:total_send])
                torch.cuda.synchronize()
                dist.barrier()
            assert np.array_equal(out[:nl[rank] + total_recv].cpu().numpy(), ref[rank]), f"{cls.__name__} forward"
            np.testing.assert_allclose(back.cpu().numpy(), refb[rank], rtol=1e-6, atol=1e-6)
            assert int(seen.item()) == 4
        e.check_status()
        dist.barrier()
        e.teardown()
        del xb, gb

    # DistGraphBuilder across real ranks: the union of the ranks' edges is the full graph, the halo
    # CSR equals the oracle's build_halo_maps for the partition the ranks agreed on
    from dynamis_b200.dist_graph_builder import BuildMode, DistGraphBuilder

    b = DistGraphBuilder(torch.as_tensor(cell, device=dev), torch.tensor([True] * 3), 6.0, 0.5, env, refresh_interval=5)
    tp = torch.as_tensor(pos, device=dev)
    gfull = O.radius_graph(pos, cell, [1, 1, 1], 6.0)
    for it in range(2):
        res = b.build(tp)
        assert res.mode == (BuildMode.REFRESH if it == 0 else BuildMode.STEADY)
        assert np.array_equal(res.full_degrees.cpu().numpy(), gfull["counts"])
        pid_b = res.pid_outer.cpu().numpy()
        assert np.array_equal(pid_b, O.sfc_partition(pos, gfull["counts"].astype(np.int64), W, 0))
        mb = O.build_halo_maps(g["src"], g["dst"], pid_b, rank, W)
        assert np.array_equal(res.halo_info.send_local_indices.cpu().numpy(), mb["send_local_indices"])
        assert np.array_equal(res.halo_recv_global_ids.cpu().numpy(), mb["recv_atom_global"])
        assert np.array_equal(res.interior_mask.cpu().numpy(), mb["interior_mask"])
        mine = O.canonical_edges(res.edges_outer[0].cpu().numpy(), res.edges_outer[1].cpu().numpy(), res.cell_shifts_outer.cpu().numpy())
        sel = pid_b[gfull["dst"]] == rank
        want = O.canonical_edges(gfull["src"][sel], gfull["dst"][sel], gfull["shift"][sel])
        assert mine.shape == want.shape and (mine == want).all(), f"DistGraphBuilder edges differ (pass {it})"
    # SimState across real ranks: atoms drift, the state is gathered, repartitioned and rebuilt
    mol = D.MolecularInfo()
    mol.num_atoms = n
    mol.atom_positions = torch.as_tensor(pos, device=dev)
    vel_np = np.random.default_rng(7).normal(0, 0.05, (n, 3)).astype(np.float32)
    mol.atom_velocities = torch.as_tensor(vel_np, device=dev)
    mol.atom_types = torch.zeros(n, dtype=torch.int64, device=dev)
    mol.atom_vertex_numbers = torch.arange(n, dtype=torch.int64, device=dev)
    cfg2 = D.SimulationConfig()
    cfg2.cutoff, cfg2.ghost_cutoff_buffer, cfg2.cell, cfg2.pbc = 6.0, 0.5, torch.as_tensor(cell), torch.tensor([True] * 3)
    env.local_rank = dev.index
    sim = D.SimState(mol, D.SFCPartitioner(), cfg2, env, device=dev)
    old_idx = sim.local_partition_info.partition_indices.clone()
    for _ in range(3):
        sim.pos.add_(sim.vel)                      # x += v, three steps
    want_pos = pos + 3 * vel_np
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    sim.write_local_drift_flag(flag, 0.25, 1.0)
    d = np.linalg.norm(3 * vel_np[old_idx.cpu().numpy()], axis=1)
    assert int(flag.item()) & 2 == (2 if d.max() > 0.25 else 0)
    sim.sync_positions_and_rebuild_halo()
    np.testing.assert_allclose(sim._state.global_molecular_info.atom_positions.cpu().numpy(), want_pos, rtol=0, atol=1e-5)
    g2 = O.radius_graph(want_pos.astype(np.float32), cell, [1, 1, 1], np.float32(6.5))
    m2 = O.build_halo_maps(g2["src"], g2["dst"], pid, rank, W)
    gp = sim._state.global_molecular_info.atom_positions.cpu().numpy()
    if np.array_equal(gp, want_pos.astype(np.float32)):
        assert np.array_equal(sim.local_partition_info.send_local_indices.cpu().numpy(), m2["send_local_indices"])
    sim.sync_and_repartition()
    gp = sim._state.global_molecular_info.atom_positions.cpu().numpy()
    gv = sim._state.global_molecular_info.atom_velocities.cpu().numpy()
    assert np.array_equal(gv, vel_np)
    pid3 = O.sfc_partition(gp, None, W, 0)
    assert np.array_equal(sim.local_partition_info.partition_id.cpu().numpy(), pid3)
    mine3 = np.nonzero(pid3 == rank)[0]
    assert np.array_equal(sim.local_partition_info.partition_indices.cpu().numpy(), mine3)
    assert np.array_equal(sim.pos.cpu().numpy(), gp[mine3]) and np.array_equal(sim.vel.cpu().numpy(), vel_np[mine3])
    g3 = O.radius_graph(gp, cell, [1, 1, 1], np.float32(6.5))
    m3 = O.build_halo_maps(g3["src"], g3["dst"], pid3, rank, W)
    assert np.array_equal(sim.local_partition_info.recv_atom_global.cpu().numpy(), m3["recv_atom_global"])
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok", flush=True)


if __name__ == "__main__":
    main()
