"""N > 1 arm of bench.py: one rank per GPU (torchrun, NCCL for the plumbing).

Default workload ("fcc", strong scaling): the 8,001,504-atom fcc Cu supercell (126^3 cells, a = 3.615 A,
jitter 0.1 A, fp32, cutoff 6 A) cut into N subdomains along the Morton curve, halo width 12 A
(ghost_cutoff_buffer 6 A).  `--workload liquid` keeps the weak-scaling liquid (N x 1,000,000 atoms,
cutoff 5 A, halo 5.5 A).  Set-up (untimed): partition, halo maps at cutoff + buffer, exchanger set-up,
and a parity check of everything the timed step does.  One timed step on every rank:

  1. forward halo push of the positions (F = 3)
  2. radius graph of the owned atoms over [owned | halo]
  3. two forward halo pushes of 128-wide node embeddings
  4. three reverse pushes with accumulation (2 x F = 128, 1 x F = 3 for the forces)

value = edges of all ranks / max-over-ranks step time (CUDA events on each rank's stream).
"""

from __future__ import annotations

import json
import time

import numpy as np
import torch
import torch.distributed as dist

import bench as B

F_EMB = 128
NVLINK_PEER_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool


def _edge_digest(edge_index: torch.Tensor, shifts: torch.Tensor, id_map=None):
    """Order-independent 64-bit digest of an edge set (count, wrapped sum of per-edge hashes)."""
    src, dst = edge_index[0], edge_index[1]
    if id_map is not None:
        src, dst = id_map[src], id_map[dst]
    sh = shifts.round().to(torch.int64) + 512
    h = src * (-7046029254386353131) + dst * (-4417276706812531889)
    h = h ^ ((sh[:, 0] << 40) | (sh[:, 1] << 20) | sh[:, 2])
    h = h * (-2960836687051489901)
    h = h ^ ((h >> 32) & 0xFFFFFFFF)
    return torch.stack([torch.tensor(src.numel(), dtype=torch.int64, device=src.device), h.sum()])


def _emb_of(gid: torch.Tensor, salt: int) -> torch.Tensor:
    """Deterministic small-integer rows of a global atom id: every rank can say what any ghost row must be."""
    f = torch.arange(F_EMB, device=gid.device, dtype=torch.int64)
    return (((gid[:, None] * 7 + f[None, :] * 3 + salt) % 17) - 8).to(torch.float32)


def _grad_of(rank: int, gid: torch.Tensor, F: int, salt: int) -> torch.Tensor:
    """Gradient rows as small integers of (holder rank, global id): their sums are exact in float32."""
    f = torch.arange(F, device=gid.device, dtype=torch.int64)
    return (((gid[:, None] * 5 + f[None, :] + rank * 13 + salt) % 11) - 5).to(torch.float32)


def run_migrate(args, rank: int, world: int, dev: torch.device):
    """--workload migrate: the 4,000,000-atom liquid (density 0.1, cutoff 5 A, buffer 0.5 A) drifting with Gaussian
    per-atom velocities (sigma 0.05 A per step) for 100 steps.  The atoms stay distributed throughout: halo maps
    are rebuilt when the largest displacement since the last rebuild reaches buffer / 2, the system is
    repartitioned along the Morton curve every 25 steps with the movers sent to their new owners, and every step
    pushes three layers of 256-wide embeddings through the current halo plan.  Reports wall-clock milliseconds
    (max over ranks) per repartition, per halo-only rebuild, per exchanger set-up and per exchange step."""
    import dynamis_b200 as D
    from dynamis_b200 import synthetic

    n_total, F, layers, steps, every = 4_000_000, 256, 3, 100, 25
    pos_np, cell_np, pbc_np, r = synthetic.random_liquid(n_total, seed=1005)
    vel_np = synthetic.drift_velocities(n_total)
    lo, hi = rank * n_total // world, (rank + 1) * n_total // world          # arbitrary first owners: blocks of ids
    env = D.DistEnvironment()
    env.global_rank, env.world_size, env.gpus_per_node, env.num_nodes, env.local_rank = rank, world, world, 1, dev.index
    cfg = D.SimulationConfig()
    cfg.cutoff, cfg.ghost_cutoff_buffer = r, 0.5
    cfg.cell, cfg.pbc = torch.from_numpy(cell_np).to(dev), torch.from_numpy(pbc_np).to(dev)
    st = D.DistributedSimState(torch.arange(lo, hi, dtype=torch.int64, device=dev), torch.from_numpy(pos_np[lo:hi]).to(dev),
                               torch.from_numpy(vel_np[lo:hi]).to(dev), None, n_total, cfg, env)
    del pos_np, vel_np

    def timed(fn):
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3

    first_ms = timed(st.repartition)                                          # nearly every atom changes owner
    ex = [D.GPUDirectExchanger(headroom=0.25) for _ in range(layers)]

    def setup():
        # with head-room the exchangers keep their peer-visible allocation and the peers' mappings of it while the
        # new plan fits: a rebuild then costs one metadata exchange per exchanger
        for x in ex:
            x.setup_exchanger(F, st.local_partition_info, dev)
            x.is_ipc_setup = True

    setup_ms = [timed(setup)]
    ref = st.pos.clone()
    rep_ms, halo_ms, push_ms, moved, ghosts = [], [], [], [], []
    for k in range(1, steps + 1):
        st.pos.add_(st.vel)
        if k % every == 0:
            rep_ms.append(timed(st.repartition))
            moved.append(st.last["atoms_leaving"])
            setup_ms.append(timed(setup))
            ref = st.pos.clone()
        else:
            far = (st.pos - ref).norm(dim=1).max().reshape(1) if st.pos.shape[0] else torch.zeros(1, device=dev)
            dist.all_reduce(far, op=dist.ReduceOp.MAX)
            if float(far) >= cfg.ghost_cutoff_buffer / 2:
                halo_ms.append(timed(st.rebuild_halo))
                setup_ms.append(timed(setup))
                ref = st.pos.clone()
        ghosts.append(int(st.local_partition_info.recv_atom_global.numel()))
        emb = torch.ones((st.pos.shape[0], F), device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        outs = [x.feature_push_forward(emb, st.local_partition_info) for x in ex]
        b.record()
        torch.cuda.synchronize()
        push_ms.append(a.elapsed_time(b))
        del outs, emb
    n_owned = torch.tensor([st.pos.shape[0]], device=dev)
    dist.all_reduce(n_owned)
    assert int(n_owned) == n_total, "atoms were lost or duplicated"

    def mx(v):
        t = torch.tensor([float(np.mean(v)) if len(v) else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    vals = [mx(rep_ms), mx(halo_ms), mx(setup_ms), mx(push_ms), mx(moved), mx(ghosts), mx([first_ms])]
    if rank == 0:
        print(json.dumps({
            "metric": "repartition_ms", "value": vals[0], "unit": "ms", "n_gpus": world, "steps": steps, "warmup": 0,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"random liquid {n_total} atoms, density 0.1, cutoff 5.0 A, buffer 0.5 A (configs[4]): 100 drift steps "
                                   f"(sigma 0.05 A/step), halo rebuild on max displacement >= buffer/2, Morton repartition every {every} "
                                   f"steps with migration, {layers} x F={F} forward pushes per step; the atoms stay distributed"},
            "repartition_ms": vals[0], "repartitions": len(rep_ms), "atoms_leaving_per_repartition_max": vals[4],
            "halo_rebuild_ms": vals[1], "halo_rebuilds": len(halo_ms), "exchanger_setup_ms": vals[2],
            "push_ms_per_step": vals[3], "halo_atoms_max": vals[5], "first_repartition_ms": vals[6],
            "timing": "wall clock around each call with a device synchronisation on both sides, mean over calls, max over ranks",
        }), flush=True)
    dist.barrier()
    for x in ex:
        x.reset_buffers()
    dist.destroy_process_group()


def run_exchange_parts(args, rank: int, world: int, dev: torch.device):
    """--workload exchange: the pieces of one forward halo push timed apart, on synthetic plans of the size
    of the fcc workload (per rank n_local rows of F = 128 floats, `send` rows spread evenly over the peers):
    stores into the peers alone, the copy of the own rows alone, both in one launch (the product), and the
    copy-engine route (pack kernel + one peer copy per rank).  CUDA events, median, max over ranks."""
    import ctypes  # noqa: F401

    import dynamis_b200 as D
    from dynamis_b200 import _lib

    n_local = 8_001_504 // world
    per = 395_000 // (world - 1)
    n_send, F = per * (world - 1), F_EMB
    rng = np.random.default_rng(rank)
    sl = np.concatenate([np.sort(rng.choice(n_local, per, replace=False)) for _ in range(world - 1)])
    cnt = np.array([0 if p == rank else per for p in range(world)])
    so = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int64)
    e = D.FeatureExchanger(result_ring=0)
    meta = e.local_setup(torch.as_tensor(so), torch.as_tensor(sl), torch.as_tensor(so.copy()), n_local, F, rank, world, dev)
    metas = [None] * world
    dist.all_gather_object(metas, meta)
    e.connect(metas)
    x = torch.randn(n_local, F, device=dev)
    out = torch.empty(n_local + n_send, F, device=dev)
    stage = torch.empty(n_send, F, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    L, rb = _lib.lib(), F * 4
    st = torch.cuda.current_stream(dev).cuda_stream

    def timed(fn):
        ts = []
        for _ in range(max(args.steps, 5)):
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        t = torch.tensor([float(np.median(ts))], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def begin(head: bool, skip: int):
        e._gen[0] += 1
        _lib.check(L.dynb_halo_forward_begin(e._ctx.ref(), x.data_ptr(), n_local, rb, e.send_local.data_ptr(), e.total_send,
                                             out.data_ptr() if head else None, e._gen[0], 0, skip, st), "halo_forward_begin")
        _lib.check(L.dynb_halo_forward_end(e._ctx.ref(), e._gen[0], e.wait_ns, None, None, 0, st), "halo_forward_end")

    def pack():
        _lib.check(L.dynb_pack_rows(x.data_ptr(), n_local, rb, e.send_local.data_ptr(), n_send, stage.data_ptr(), None, st), "pack_rows")

    def peer_copies():
        for r in e._peer_recs:
            if r.remote_base:
                _lib.check(L.dynb_copy_async(r.remote_base + r.fwd_stage_off[0] + r.fwd_row_offset * rb,
                                             stage.data_ptr() + r.send_start * rb, r.send_count * rb, st), "copy_async")

    res = {"push_only_ms": timed(lambda: begin(False, 0)), "push_only_in_list_order_ms": timed(lambda: begin(False, 2)),
           "copy_only_ms": timed(lambda: begin(True, 1)), "push_and_copy_ms": timed(lambda: begin(True, 0)),
           "push_and_copy_in_list_order_ms": timed(lambda: begin(True, 2)), "pack_ms": timed(pack),
           "peer_copies_ms": timed(peer_copies)}
    e.check_status()
    if rank == 0:
        mb = n_send * rb / 1e6
        print(json.dumps({"metric": "halo_push_parts_ms", "n_gpus": world, "rows_local": n_local, "rows_sent": n_send, "F": F,
                          "payload_mb_per_rank": mb, "copy_gb_per_rank": 2 * n_local * rb / 1e9, **res,
                          "push_only_gbs": mb / res["push_only_ms"], "peer_copies_gbs": mb / res["peer_copies_ms"],
                          "timing": "CUDA events on each rank's stream, L2 flushed, median, max over ranks; each piece is "
                                    "followed by the bounded wait for all peers' signals where it signals"}), flush=True)
    dist.barrier()
    e.teardown()
    dist.destroy_process_group()


def run(args, rank: int, world: int, dev: torch.device):
    import dynamis_b200 as D
    from dynamis_b200 import synthetic

    if args.workload == "migrate":
        return run_migrate(args, rank, world, dev)
    if args.workload == "exchange":
        return run_exchange_parts(args, rank, world, dev)
    K, Wm = args.steps, max(args.warmup, 3)
    if args.workload == "liquid":
        n_total = B.ATOMS_PER_GPU * world
        pos_np, cell_np, pbc_np, r = B.liquid(n_total)
        halo_buffer, scaling = 0.5, "weak"
        wl = (f"random liquid {n_total} atoms ({B.ATOMS_PER_GPU}/GPU), density 0.1, fp32, cutoff 5.0 A, Morton partition into "
              f"{world} subdomains, halo {r + halo_buffer} A")
    else:
        pos_np, cell_np, pbc_np, r = synthetic.fcc_copper(126, seed=1004)
        n_total = pos_np.shape[0]
        halo_buffer, scaling = 6.0, "strong"
        wl = (f"fcc Cu {n_total} atoms (126^3 cells, a=3.615 A, jitter 0.1 A, fp32), cutoff 6.0 A (configs[3]), Morton partition "
              f"into {world} subdomains, halo {r + halo_buffer} A")
    pos_g = torch.from_numpy(pos_np).to(dev)
    cell = torch.from_numpy(cell_np)
    pbc = torch.from_numpy(pbc_np)

    st = D.MolecularInfo()
    st.num_atoms = n_total
    st.atom_positions = pos_g
    st.atom_vertex_numbers = torch.arange(n_total, dtype=torch.int64, device=dev)
    env = D.DistEnvironment()
    env.global_rank, env.world_size, env.gpus_per_node, env.num_nodes, env.local_rank = rank, world, world, 1, dev.index
    cfg = D.SimulationConfig()
    cfg.cutoff, cfg.ghost_cutoff_buffer, cfg.cell, cfg.pbc = r, halo_buffer, cell, pbc

    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats(dev)
    t0 = time.perf_counter()
    part = D.SFCPartitioner()
    info = part.partition(st, env)
    part.build_halo_maps(info, st, env, cfg)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t0
    setup_peak_gb = torch.cuda.max_memory_allocated(dev) / 1e9
    n_local = info.partition_indices.numel()
    n_ghost = info.recv_atom_global.numel()
    total_send = int(info.send_offsets[-1].item())
    state = D.DynamisState()
    state.local_partition_info = info

    mk = (lambda: D.GPUDirectExchanger()) if args.exchange == "peer" else (lambda: D.PythonNCCLExchanger())
    ex_pos, ex_e1, ex_e2 = mk(), mk(), mk()
    if args.exchange == "peer" and args.ce_threshold > 0:
        for x in (ex_pos, ex_e1, ex_e2):
            x.exchanger.set_ce_threshold_bytes(args.ce_threshold)

    mine = info.partition_indices
    ghosts = info.recv_atom_global
    pos_local = pos_g[mine].contiguous()
    emb1, emb2 = _emb_of(mine, 1), _emb_of(mine, 2)
    targets = torch.arange(n_local, dtype=torch.int64, device=dev)
    gid_all = torch.cat([mine, ghosts])
    g_emb1, g_emb2 = _grad_of(rank, gid_all, F_EMB, 1), _grad_of(rank, gid_all, F_EMB, 2)
    g_pos = _grad_of(rank, gid_all, 3, 3)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def step(p_local, timers=None):
        e = [ev() for _ in range(8)] if timers is not None else None
        if e: e[0].record()
        allpos = ex_pos.feature_push_forward(p_local, info)
        if e: e[1].record()
        out = D.radius_graph_pbc_ex(allpos, cell, pbc, r, 0, False, targets)
        if e: e[2].record()
        h1 = ex_e1.feature_push_forward(emb1, info)
        if e: e[3].record()
        h2 = ex_e2.feature_push_forward(emb2, info)
        if e: e[4].record()
        b2 = ex_e2.feature_push_backward(g_emb2, emb2.shape, info)
        if e: e[5].record()
        b1 = ex_e1.feature_push_backward(g_emb1, emb1.shape, info)
        if e: e[6].record()
        f = ex_pos.feature_push_backward(g_pos, p_local.shape, info)
        if e:
            e[7].record()
            timers.append(e)
        return out, (allpos, h1, h2, b1, b2, f)

    # ---- parity of one whole step, before anything is timed --------------------------------------------------
    out, (allpos, h1, h2, b1, b2, f) = step(pos_local)
    ok = {}
    ok["ghost_positions"] = bool(torch.equal(allpos[n_local:], pos_g[ghosts]) and torch.equal(allpos[:n_local], pos_local))
    ok["ghost_embeddings"] = bool(torch.equal(h1, _emb_of(gid_all, 1)) and torch.equal(h2, _emb_of(gid_all, 2)))
    # reverse: an owned row receives, from every peer p that holds it as a ghost, the gradient row p made for it
    so = info.send_offsets.cpu().tolist()
    sl = info.send_local_indices

    def reverse_expected(g_local, F, salt):
        want = g_local[:n_local].clone()
        for p in range(world):
            if p == rank or so[p + 1] == so[p]:
                continue
            rows = sl[so[p]:so[p + 1]]
            want.index_add_(0, rows, _grad_of(p, mine[rows], F, salt))
        return want

    ok["reverse_embeddings"] = bool(torch.equal(b1, reverse_expected(g_emb1, F_EMB, 1)) and
                                    torch.equal(b2, reverse_expected(g_emb2, F_EMB, 2)))
    ok["reverse_forces"] = bool(torch.equal(f, reverse_expected(g_pos, 3, 3)))
    # edges: the ranks' owned-atom graphs together are the graph of the whole system (count and digest)
    dg = _edge_digest(out[0], out[1], gid_all)
    dist.all_reduce(dg, op=dist.ReduceOp.SUM)
    E_local = int(out[2].item())
    del out, allpos, h1, h2, b1, b2, f
    full = D.radius_graph_pbc_ex(pos_g, cell, pbc, r, 0, False) if rank == 0 else None
    if rank == 0:
        dfull = _edge_digest(full[0], full[1])
        ok["edge_union_vs_single_rank"] = bool(torch.equal(dfull, dg))
        del full
    flags = torch.tensor([int(all(ok.values()))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if int(flags.item()) != 1:
        print(json.dumps({"rank": rank, "parity_failed": ok}), flush=True)
        dist.barrier()
        raise SystemExit(3)
    del pos_g, st
    torch.cuda.empty_cache()

    for _ in range(Wm):
        out, _x = step(pos_local)
    del out, _x
    torch.cuda.synchronize()
    dist.barrier()

    sampler = B.ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    tw0 = time.perf_counter()
    tot_ms = exch_ms = graph_ms = 0.0
    parts = np.zeros(6)
    for _ in range(K):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        timers = []
        out, _x = step(pos_local, timers)
        torch.cuda.synchronize()
        e = timers[0]
        tot_ms += e[0].elapsed_time(e[7])
        graph_ms += e[1].elapsed_time(e[2])
        exch_ms += e[0].elapsed_time(e[1]) + e[2].elapsed_time(e[7])
        parts += np.array([e[0].elapsed_time(e[1])] + [e[i].elapsed_time(e[i + 1]) for i in range(2, 7)])
        del out, _x
    tw1 = time.perf_counter()
    clocks = sampler.stop(tw0, tw1) if rank == 0 else None
    for x in (ex_pos, ex_e1, ex_e2):
        if hasattr(x, "exchanger"):
            x.exchanger.check_status()

    # the two launches of one exchange apart (first: push + own rows + signal; second: wait + what needs the peers' rows)
    halves = np.zeros(4)
    if args.exchange == "peer":
        fe = ex_e1.exchanger
        for _ in range(K):
            torch.cuda.synchronize()
            dist.barrier()
            e = [ev() for _ in range(6)]
            e[0].record()
            o, gen = fe.forward_begin(emb1)
            e[1].record()
            o = fe.forward_end(o, gen)
            e[2].record()
            e[3].record()
            gb, gen = fe.backward_begin(g_emb1)
            e[4].record()
            gb = fe.backward_end(gb, gen)
            e[5].record()
            torch.cuda.synchronize()
            halves += np.array([e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), e[3].elapsed_time(e[4]), e[4].elapsed_time(e[5])])
            del o, gb

    # end to end: local positions from pinned host memory, degrees + edge count back
    pos_pin = pos_local.cpu().pin_memory()
    counts_pin = torch.empty(n_local, dtype=torch.int32).pin_memory()
    nni_pin = torch.empty(1, dtype=torch.int64).pin_memory()
    p_in = torch.empty_like(pos_local)
    torch.cuda.synchronize()
    dist.barrier()
    te0 = time.perf_counter()
    for _ in range(K):
        p_in.copy_(pos_pin, non_blocking=True)
        out, _x = step(p_in)
        counts_pin.copy_(out[3], non_blocking=True)
        nni_pin.copy_(out[2], non_blocking=True)
        torch.cuda.synchronize()
        del out, _x
    dist.barrier()
    e2e_s = (time.perf_counter() - te0) / K

    # the dominant kernel alone on this rank's graph (edge-writing pass), as in the single-GPU arm
    from dynamis_b200 import graph as G

    allpos = ex_pos.feature_push_forward(pos_local, info)
    plan = G.plan_radius_graph(allpos, cell, pbc, r, targets)
    ei = torch.empty((2, plan.E), dtype=torch.int64, device=dev)
    sh = torch.empty((plan.E, 3), dtype=torch.float32, device=dev)
    plan.fill_into(ei, sh)
    torch.cuda.synchronize()
    kt = []
    for _ in range(10):
        flush.zero_()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        plan.fill_into(ei, sh)
        b.record()
        torch.cuda.synchronize()
        kt.append(a.elapsed_time(b))
    fill_ms = float(np.mean(kt))
    del ei, sh, allpos
    peak, peak_kind = B._peaks()

    red = torch.tensor([tot_ms / K, exch_ms / K, graph_ms / K, e2e_s * 1e3] + list(parts / K) + list(halves / K),
                       device=dev, dtype=torch.float64)
    red_min = red.clone()
    dist.all_reduce(red, op=dist.ReduceOp.MAX)
    dist.all_reduce(red_min, op=dist.ReduceOp.MIN)
    sums = torch.tensor([E_local, n_local, n_ghost, total_send], device=dev, dtype=torch.int64)
    mx = sums.clone()
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    if rank == 0:
        v, vmin = [float(x) for x in red.tolist()], [float(x) for x in red_min.tolist()]
        ms, xms, gms, ems = v[:4]
        E_total = int(sums[0])
        # bytes one rank sends per step: forward 3 + 128 + 128 floats per sent row, reverse the same per ghost row
        bytes_rank = (int(mx[3]) + int(mx[2])) * (3 + 2 * F_EMB) * 4
        names = ["fwd_pos_F3", "fwd_emb1_F128", "fwd_emb2_F128", "bwd_emb2_F128", "bwd_emb1_F128", "bwd_pos_F3"]
        line = {
            "metric": "radius_graph_edges_per_s", "value": E_total / (ms * 1e-3), "unit": "edges/s", "n_gpus": world,
            "steps": K, "warmup": Wm, "ms_per_step": ms, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl + f": per step 1 position push (F=3), owned-atom radius graph over [owned|halo], 2 embedding "
                                     f"pushes (F={F_EMB}), 3 reverse pushes (the N = 1 line is configs[1], radius graph + Morton "
                                     "partition without exchange)",
                       "edges_per_step": E_total, "exchange": args.exchange, "ce_threshold_bytes": args.ce_threshold,
                       "atoms_local_max": int(mx[1]), "halo_atoms_max": int(mx[2]), "send_rows_max": int(mx[3]),
                       "l2": "256 MiB buffer written between timed steps", "setup_s": setup_s,
                       "setup_peak_gb": setup_peak_gb},
            "parity_checked": {"ok": True, "checks": sorted(ok), "how": "untimed first step on every rank: ghost rows equal the "
                               "owners' rows bit for bit, reverse-accumulated rows equal index_add_ of the peers' rows (integer-valued "
                               "gradients, exact), ranks' edge sets together equal a single-rank build (count + 64-bit digest)"},
            "halo_exchange_ms_per_step": xms, "graph_ms_per_step": gms,
            "graph_edges_per_s": E_total / (gms * 1e-3),
            "exchange_breakdown": {"ms_max_over_ranks": dict(zip(names, v[4:10])), "ms_min_over_ranks": dict(zip(names, vmin[4:10])),
                                   "emb_push_halves_ms_max": dict(zip(["fwd_begin", "fwd_end", "bwd_begin", "bwd_end"], v[10:14])),
                                   "emb_push_halves_ms_min": dict(zip(["fwd_begin", "fwd_end", "bwd_begin", "bwd_end"], vmin[10:14]))},
            "nvlink": {"bytes_sent_per_rank_per_step": bytes_rank, "achieved_gbs": bytes_rank / (xms * 1e-3) / 1e9,
                       "peak_gbs": NVLINK_PEER_GBS, "peak_kind": "measured peer copy per direction",
                       "frac": bytes_rank / (xms * 1e-3) / 1e9 / NVLINK_PEER_GBS},
            "roofline": {"bound": "hbm", "kernel": "rg_fillmask_kernel<float> (rank 0)", "achieved": 28.0 * plan.E / (fill_ms * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": 28.0 * plan.E / (fill_ms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind,
                         "traffic": None, "algorithmic_bytes": 28.0 * plan.E, "ms_per_launch": fill_ms},
            "cpu_baseline": None,
            "e2e": {"value": E_total / (ems * 1e-3), "unit": "edges/s", "ms_per_step": ems,
                    "h2d_bytes_per_step": int(sums[1]) * 12, "d2h_bytes_per_step": int(sums[1]) * 4 + 8 * world,
                    "note": "positions in from pinned host memory, degrees and edge count out; the edge list stays on the device, "
                            "as with the API it replaces (CUDA tensors for a CUDA consumer)"},
            "clocks": clocks,
            "gpu_launches": D.launches_per_graph(target_subset=True) + 6 * 2,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    for x in (ex_pos, ex_e1, ex_e2):
        x.reset_buffers()
    dist.destroy_process_group()
