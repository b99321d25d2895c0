"""N > 1 arm of bench.py: one rank per GPU (torchrun, NCCL for the plumbing).

Workload (weak scaling of the single-GPU workload): the random liquid with N x 1,000,000 atoms
(density 0.1 atoms/A^3, fp32, cutoff 5 A), cut into N subdomains along the Morton curve.  Set-up
(untimed): partition, halo maps at cutoff + buffer, exchanger set-up.  One timed step on every rank:

  1. forward halo push of the positions (F = 3)
  2. radius graph of the owned atoms over [owned | halo]
  3. two forward halo pushes of 128-wide node embeddings
  4. three reverse pushes with accumulation (2 x F = 128, 1 x F = 3 for the forces)

value = edges of all ranks / max-over-ranks step time (CUDA events on each rank's stream).
"""

from __future__ import annotations

import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

import bench as B

HALO_BUFFER = float(os.environ.get("DYNB_BENCH_HALO_BUFFER", "0.5"))
F_EMB = 128
NVLINK_PEER_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool


def run(args, rank: int, world: int, dev: torch.device):
    import dynamis_b200 as D

    K, Wm = args.steps, max(args.warmup, 3)
    n_total = B.ATOMS_PER_GPU * world
    pos_np, cell_np, pbc_np, r = B.liquid(n_total)
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
    cfg.cutoff, cfg.ghost_cutoff_buffer, cfg.cell, cfg.pbc = r, HALO_BUFFER, cell, pbc

    t0 = time.perf_counter()
    part = D.SFCPartitioner()
    info = part.partition(st, env)
    part.build_halo_maps(info, st, env, cfg)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t0
    n_local = info.partition_indices.numel()
    n_ghost = info.recv_atom_global.numel()
    total_send = int(info.send_offsets[-1].item())
    state = D.DynamisState()
    state.local_partition_info = info

    kind = os.environ.get("DYNB_BENCH_EXCHANGE", "peer")
    mk = (lambda: D.GPUDirectExchanger()) if kind == "peer" else (lambda: D.PythonNCCLExchanger())
    ex_pos, ex_e1, ex_e2 = mk(), mk(), mk()

    pos_local = pos_g[info.partition_indices].contiguous()
    del pos_g, st
    emb1 = torch.randn((n_local, F_EMB), device=dev, generator=torch.Generator(device=dev).manual_seed(2004 + rank))
    emb2 = torch.randn((n_local, F_EMB), device=dev, generator=torch.Generator(device=dev).manual_seed(3004 + rank))
    targets = torch.arange(n_local, dtype=torch.int64, device=dev)
    g_emb = torch.ones((n_local + n_ghost, F_EMB), device=dev)
    g_pos = torch.ones((n_local + n_ghost, 3), device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def step(p_local, timers=None):
        e = [ev() for _ in range(4)] if timers is not None else None
        if e: e[0].record()
        allpos = ex_pos.feature_push_forward(p_local, info)
        if e: e[1].record()
        out = D.radius_graph_pbc_ex(allpos, cell, pbc, r, 0, False, targets)
        if e: e[2].record()
        h1 = ex_e1.feature_push_forward(emb1, info)
        h2 = ex_e2.feature_push_forward(emb2, info)
        b2 = ex_e2.feature_push_backward(g_emb, emb2.shape, info)
        b1 = ex_e1.feature_push_backward(g_emb, emb1.shape, info)
        f = ex_pos.feature_push_backward(g_pos, p_local.shape, info)
        if e:
            e[3].record()
            timers.append(e)
        return out, (h1, h2, b1, b2, f)

    for _ in range(Wm):
        out, _x = step(pos_local)
    E_local = int(out[2].item())
    del out, _x
    torch.cuda.synchronize()
    dist.barrier()

    sampler = B.ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    tw0 = time.perf_counter()
    tot_ms = exch_ms = graph_ms = 0.0
    for _ in range(K):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        timers = []
        out, _x = step(pos_local, timers)
        torch.cuda.synchronize()
        e = timers[0]
        tot_ms += e[0].elapsed_time(e[3])
        graph_ms += e[1].elapsed_time(e[2])
        exch_ms += e[0].elapsed_time(e[1]) + e[2].elapsed_time(e[3])
        del out, _x
    tw1 = time.perf_counter()
    clocks = sampler.stop(tw0, tw1) if rank == 0 else None
    for x in (ex_pos, ex_e1, ex_e2):
        if hasattr(x, "exchanger"):
            x.exchanger.check_status()

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
    del ei, sh
    peak, peak_kind = B._peaks()

    red = torch.tensor([tot_ms / K, exch_ms / K, graph_ms / K, e2e_s * 1e3], device=dev, dtype=torch.float64)
    dist.all_reduce(red, op=dist.ReduceOp.MAX)
    sums = torch.tensor([E_local, n_local, n_ghost, total_send], device=dev, dtype=torch.int64)
    mx = sums.clone()
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms, xms, gms, ems = [float(v) for v in red.tolist()]
        E_total = int(sums[0])
        # bytes one rank sends per step: forward 3 + 128 + 128 floats per sent row, reverse the same per ghost row
        bytes_rank = (int(mx[3]) + int(mx[2])) * (3 + 2 * F_EMB) * 4
        line = {
            "metric": "radius_graph_edges_per_s", "value": E_total / (ms * 1e-3), "unit": "edges/s", "n_gpus": world,
            "steps": K, "warmup": Wm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"random liquid {n_total} atoms ({B.ATOMS_PER_GPU}/GPU), density 0.1, fp32, cutoff 5.0 A, "
                                   f"Morton partition into {world} subdomains, halo {r + HALO_BUFFER} A: per step 1 position push (F=3), "
                                   f"owned-atom radius graph over [owned|halo], 2 embedding pushes (F={F_EMB}), 3 reverse pushes "
                                   "(the N = 1 step is radius graph + Morton sort and has no exchange: compare graph_edges_per_s across N)",
                       "edges_per_step": E_total, "exchange": kind, "atoms_local_max": int(mx[1]), "halo_atoms_max": int(mx[2]),
                       "l2": "256 MiB buffer written between timed steps", "setup_s": setup_s},
            "halo_exchange_ms_per_step": xms, "graph_ms_per_step": gms,
            # the two halves of the metric ("radius-graph edges/s and per-step halo-exchange latency") separately:
            # `value` divides by the whole step, which at N > 1 also holds six halo exchanges that the N = 1 step
            # (radius graph + Morton sort, no peers) does not have
            "graph_edges_per_s": E_total / (gms * 1e-3),
            "nvlink": {"bytes_sent_per_rank_per_step": bytes_rank, "achieved_gbs": bytes_rank / (xms * 1e-3) / 1e9,
                       "peak_gbs": NVLINK_PEER_GBS, "peak_kind": "measured peer copy per direction",
                       "frac": bytes_rank / (xms * 1e-3) / 1e9 / NVLINK_PEER_GBS},
            "roofline": {"bound": "hbm", "kernel": "rg_fillmask_kernel<float> (rank 0)", "achieved": 28.0 * plan.E / (fill_ms * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": 28.0 * plan.E / (fill_ms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind,
                         "traffic": None, "algorithmic_bytes": 28.0 * plan.E, "ms_per_launch": fill_ms},
            "cpu_baseline": None,
            "e2e": {"value": E_total / (ems * 1e-3), "unit": "edges/s", "ms_per_step": ems,
                    "h2d_bytes_per_step": int(sums[1]) * 12, "d2h_bytes_per_step": int(sums[1]) * 4 + 8 * world},
            "clocks": clocks,
            "gpu_launches": D.launches_per_graph() + 6 * 4,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    for x in (ex_pos, ex_e1, ex_e2):
        x.reset_buffers()
    dist.destroy_process_group()
