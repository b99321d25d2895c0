"""Worker for test_migrate_gpu.py (torchrun).  W ranks hold an arbitrary split of a periodic system;
DistributedSimState repartitions it along the curve, migrates the atoms and rebuilds the halo maps without
any rank holding the whole system.  Everything is compared with the CPU oracle's partition of the
gathered system and its build_halo_maps — the results of the reference's replicated
sync_and_repartition / sync_positions_and_rebuild_halo (dynamis/src/dynamis/simulatorState.py:136-246).

With fewer GPUs than ranks the ranks share cuda:0 and the collectives go over gloo (no kernel of one rank
ever waits for another rank's kernel here: the only cross-rank steps are host-side collectives)."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import dynamis_b200 as D  # noqa: E402
from dynamis_b200.migrate import DistributedSimState  # noqa: E402
from oracle import cpu_oracle as O  # noqa: E402


def check(st, rank, W, pos, vel, cell, pbc, reach, curve, pid, what):
    mine = np.nonzero(pid == rank)[0]
    assert np.array_equal(st.gid.cpu().numpy(), mine), f"{what}: owned ids"
    assert np.array_equal(st.pos.cpu().numpy(), pos[mine]), f"{what}: owned positions"
    assert np.array_equal(st.vel.cpu().numpy(), vel[mine]), f"{what}: owned velocities"
    g = O.radius_graph(pos, cell, pbc, np.float32(reach))
    m = O.build_halo_maps(g["src"], g["dst"], pid, rank, W)
    info = st.local_partition_info
    for name in ("send_offsets", "send_local_indices", "recv_offsets", "recv_atom_global", "interior_mask"):
        assert np.array_equal(getattr(info, name).cpu().numpy(), m[name]), f"{what}: {name}"
    assert np.array_equal(info.partition_indices.cpu().numpy(), mine)
    assert np.array_equal(info.recv_ghost_indices.cpu().numpy(), np.arange(mine.size, mine.size + m["recv_atom_global"].size))


def main():
    rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    shared = torch.cuda.device_count() < W
    dev = torch.device("cuda", 0 if shared else int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    if shared:
        dist.init_process_group("gloo")
    else:
        dist.init_process_group("nccl", device_id=dev)
    env = D.DistEnvironment()
    env.global_rank, env.world_size, env.local_rank = rank, W, dev.index

    cases = [
        # name, N, cell, cutoff, buffer, curve
        ("cubic/morton", 24_000, np.eye(3) * 62.0, 5.0, 0.5, 0),
        ("cubic/hilbert", 12_000, np.eye(3) * 50.0, 5.0, 0.5, 1),
        ("triclinic/morton", 15_000, np.array([[52.0, 0, 0], [10.4, 50.0, 0], [5.2, 0, 48.0]]), 6.0, 1.0, 0),
    ]
    for name, N, cell, rc, buf, curve in cases:
        rng = np.random.default_rng(1000 + N)
        cell = cell.astype(np.float32)
        pos = (rng.random((N, 3)) @ cell.astype(np.float64)).astype(np.float32)
        pos += rng.normal(0, 0.3, pos.shape).astype(np.float32)          # some atoms outside the cell
        vel = rng.normal(0, 0.05, (N, 3)).astype(np.float32)
        types = rng.integers(0, 3, N)
        cfg = D.SimulationConfig()
        cfg.cutoff, cfg.ghost_cutoff_buffer = rc, buf
        cfg.cell, cfg.pbc = torch.as_tensor(cell, device=dev), torch.tensor([True, True, True], device=dev)
        # arbitrary initial owners (blocks of ids), unrelated to space: nearly every atom migrates
        start = rng.permutation(N) % W if False else (np.arange(N) * 7919 % N) * W // N
        mine0 = np.nonzero(start == rank)[0]
        st = DistributedSimState(torch.as_tensor(mine0, device=dev), torch.as_tensor(pos[mine0], device=dev),
                                 torch.as_tensor(vel[mine0], device=dev), torch.as_tensor(types[mine0], device=dev), N, cfg, env,
                                 curve_type=curve)
        st.repartition()
        pid = O.sfc_partition(pos, None, W, curve)
        check(st, rank, W, pos, vel, cell, [1, 1, 1], rc + buf, curve, pid, f"{name}: repartition")
        assert np.array_equal(st.types.cpu().numpy(), types[pid == rank])
        # drift, halo-only rebuild (owners stay)
        st.pos.add_(st.vel * 3.0)
        pos = (pos + vel * np.float32(3.0)).astype(np.float32)
        st.rebuild_halo()
        check(st, rank, W, pos, vel, cell, [1, 1, 1], rc + buf, curve, pid, f"{name}: halo rebuild")
        # second repartition: now only atoms near the cuts change owner
        st.repartition()
        pid2 = O.sfc_partition(pos, None, W, curve)
        check(st, rank, W, pos, vel, cell, [1, 1, 1], rc + buf, curve, pid2, f"{name}: second repartition")
        moved = int((pid2 != pid).sum())
        tot = torch.tensor([st.last["atoms_leaving"]], dtype=torch.int64, device="cpu" if shared else dev)
        dist.all_reduce(tot)
        assert int(tot) == moved, (int(tot), moved)
        # weighted cut (the reference's mode for degree-balanced partitions): every rank passes the degrees of the
        # atoms it holds; owners and halo maps must equal those of the gathered system's weighted partition
        if name != "triclinic/morton":
            deg = O.radius_graph(pos, cell, [1, 1, 1], np.float32(rc))["counts"].astype(np.int64)
            st.repartition(weights=torch.as_tensor(deg[st.gid.cpu().numpy()], device=dev))
            pid3 = O.sfc_partition(pos, deg, W, curve)
            check(st, rank, W, pos, vel, cell, [1, 1, 1], rc + buf, curve, pid3, f"{name}: weighted repartition")
        # the halo plan drives a real exchange of the owned rows: ghost rows equal the owners' rows
        if not shared:
            ex = D.GPUDirectExchanger(wait_ns=10_000_000_000)
            out = ex.feature_push_forward(st.pos, st.local_partition_info)
            want = pos[np.concatenate([st.gid.cpu().numpy(), st.local_partition_info.recv_atom_global.cpu().numpy()])]
            assert np.array_equal(out.cpu().numpy(), want)
            dist.barrier()
            ex.reset_buffers()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok", flush=True)


if __name__ == "__main__":
    main()
