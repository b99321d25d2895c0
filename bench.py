#!/usr/bin/env python
"""Benchmark of the hot path: periodic radius graph (+ Morton partition, + halo exchange when N > 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload fcc|liquid] [--exchange peer|nccl] [--ce-threshold BYTES]      (N > 1 only)

N > 1 is launched by torchrun (one rank per GPU, NCCL).  Prints ONE JSON line on rank 0.

A "step" is one pass of the path over one batch of synthetic input:
  N = 1   the 1,000,000-atom random liquid (density 0.1 atoms/Å^3, L = 215.4 Å, fp32, r = 5 Å):
          Morton-key partition + radius graph (edge_index, shifts, degrees).
  N > 1   the 8,001,504-atom fcc Cu supercell (fp32, r = 6 Å, halo 12 Å) cut into N subdomains along
          the Morton curve (strong scaling); every rank exchanges halo positions, builds the graph
          of its own atoms over [owned | halo], then exchanges two layers of 128-wide node
          embeddings forward and the three gradients backward.  Before anything is timed one whole
          step is checked on every rank (ghost rows, reverse sums, union of the edge sets) and the
          run exits non-zero on a mismatch.  --workload liquid: N x 1,000,000 atoms of the liquid
          (weak scaling).

value       whole-job edges/s with inputs resident in HBM, CUDA-event time, max over ranks.
e2e         the same through the public API with the positions arriving from pinned host memory
            and the degrees + edge count read back every step (wall clock around the K steps).
roofline    the dominant kernel (the edge-writing pass of the cell scan) timed alone, against the
            measured HBM copy bandwidth of MEASURED_PEAKS.json.
cpu_baseline / --impl reference
            the CPU restatement of the reference's algorithm (oracle/, OpenMP over all host
            threads) on the same workload (at N > 1: rank 0's share of it); the reference itself
            has no CPU radius-graph path.
reference_cuda (N = 1)
            the reference's own CUDA kernels, compiled for sm_100 by oracle/build_ref.py, timed on
            the same inputs and GPU outside every timed region of this implementation.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ATOMS_PER_GPU = 1_000_000
DENSITY = 0.1
RADIUS = 5.0
SEED = 1002


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.samples:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm, smx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            mx = smx
            if t0 - 0.05 <= ts <= t1 + 0.15:
                mhz.append(sm)
                for nm, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        if not mhz:
            mhz = [float(l.split(",")[0]) for _, l in self.samples[-3:] if l and l.split(",")[0].strip().replace(".", "").isdigit()]
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons)}


def liquid(n_atoms: int):
    from dynamis_b200 import synthetic

    return synthetic.random_liquid(n_atoms, density=DENSITY, seed=SEED, radius=RADIUS)


def host_threads() -> int:
    """Threads the CPU arm uses: every core this process may run on (launchers such as torchrun export
    OMP_NUM_THREADS=1, so the count is passed to the oracle explicitly)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_baseline(sample_atoms: int, steps: int = 1):
    """Oracle (CPU port of the reference algorithm) on a liquid of `sample_atoms` atoms, all host threads."""
    from oracle import cpu_oracle as O

    pos, cell, pbc, r = liquid(sample_atoms)
    threads = host_threads()
    best = None
    E = 0
    for _ in range(max(1, steps)):
        t = time.perf_counter()
        g = O.radius_graph(pos, cell, pbc, r, nthreads=threads)
        dt = time.perf_counter() - t
        E = g["E"]
        best = dt if best is None else min(best, dt)
    return {"value": E / best, "unit": "edges/s", "cores": threads, "kind": "port",
            "sample": f"{sample_atoms} atoms of the same liquid (density {DENSITY}, r = {RADIUS}), {E} edges, best of {max(1, steps)}"}, best


def reference_workload(n_gpus: int, workload: str):
    """What the CPU arm computes: at N = 1 the whole single-GPU workload; at N > 1 rank 0's share of the
    N-GPU workload — the graph of the atoms rank 0 owns over [owned | atoms within the halo width of its
    bounding box] (a superset of its halo, so the edges are those of the whole-system graph)."""
    from oracle import cpu_oracle as O

    if n_gpus <= 1:
        pos, cell, pbc, r = liquid(ATOMS_PER_GPU)
        return pos, cell, pbc, r, None, ("random liquid 1,000,000 atoms, density 0.1 atoms/A^3, cubic periodic box L=215.4 A, fp32, "
                                         "cutoff 5.0 A (configs[1]): radius graph of all atoms")
    if workload == "liquid":
        pos, cell, pbc, r = liquid(ATOMS_PER_GPU * n_gpus)
        halo, name = r + 0.5, f"random liquid {ATOMS_PER_GPU * n_gpus} atoms, cutoff 5.0 A"
    else:
        from dynamis_b200 import synthetic

        pos, cell, pbc, r = synthetic.fcc_copper(126, seed=1004)
        halo, name = r + 6.0, f"fcc Cu {pos.shape[0]} atoms, cutoff 6.0 A (configs[3])"
    labels = O.sfc_partition(pos, None, n_gpus, 0)
    own = np.nonzero(labels == 0)[0]
    L = np.diag(cell).astype(np.float64)
    p64 = pos.astype(np.float64)
    w = p64  # not wrapped: a subdomain is compact in the coordinates the curve was built on
    lo, hi = w[own].min(axis=0), w[own].max(axis=0)
    keep = np.ones(pos.shape[0], dtype=bool)
    for k in range(3):
        centre, half = (lo[k] + hi[k]) / 2, (hi[k] - lo[k]) / 2
        d = np.abs(((w[:, k] - centre + L[k] / 2) % L[k]) - L[k] / 2) - half
        keep &= d <= halo
    keep[own] = True
    idx = np.nonzero(keep)[0]
    sub = pos[idx]
    targets = np.searchsorted(idx, own).astype(np.int64)
    return sub, cell, pbc, r, targets, (f"{name}, Morton partition into {n_gpus}: rank 0's share, graph of its {own.size} owned atoms "
                                        f"over {idx.size} positions (owned + everything within {halo} A of their bounding box)")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_oracle as O

    threads = host_threads()
    pos, cell, pbc, r, targets, what = reference_workload(args.gpus, args.workload)
    E = 0
    for _ in range(min(args.warmup, 1)):  # page in, build
        E = O.radius_graph(pos, cell, pbc, r, targets=targets, nthreads=threads)["E"]
    t0 = time.perf_counter()
    for _ in range(args.steps):
        E = O.radius_graph(pos, cell, pbc, r, targets=targets, nthreads=threads)["E"]
    dt = time.perf_counter() - t0
    v = E * args.steps / dt
    line = {
        "impl": "reference", "metric": "radius_graph_edges_per_s", "value": v, "unit": "edges/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if (args.gpus <= 1 or args.workload == "liquid") else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": what, "edges_per_step": E},
        "cpu_baseline": {"value": v, "unit": "edges/s", "cores": threads, "kind": "port",
                         "sample": f"{E} edges per step, {args.steps} steps"},
        "e2e": {"value": v, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU radius-graph path (radius_graph.cpp requires CUDA tensors); this is the CPU restatement of "
                "its algorithm (oracle/), OpenMP over all host threads; a CPU's edges/s does not depend on how many GPUs the "
                "other arm uses, so at N > 1 one rank's share of the job is timed",
    }
    print(json.dumps(line), flush=True)


def reference_cuda(pos, cell, pbc, r, E):
    """The reference's own CUDA kernels (compiled for sm_100 from its sources by oracle/build_ref.py) on the
    same inputs and the same GPU, outside every timed region of this implementation: the bar this
    implementation is measured against.  None when that library was not built."""
    import torch

    from oracle import build_ref

    if not build_ref.load():
        return None
    ops = torch.ops.dynamis_ref
    cell_d, pbc_d = cell.to(pos.device), pbc.to(pos.device)

    def med(fn, warm=5, reps=20):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return float(np.median(ts))

    g = med(lambda: ops.radius_graph(pos, cell_d, pbc_d, r, None, False))
    s = med(lambda: ops.sfc_partition(pos, None, 8, 0))
    k = med(lambda: ops.kdtree_partition(pos, None, 8))
    return {"graph_ms": g, "sfc_ms": s, "kdtree_ms": k, "edges_per_s": E / ((g + s) * 1e-3),
            "what": "reference CUDA kernels (radius_graph_pbc_cuda_impl_ex, sfc_partition_cuda_impl, kdtree_bisect_cuda_impl) "
                    "compiled for sm_100, CUDA events, median of 20 after 5 warm-up calls; edges_per_s over graph + Morton partition"}


def run_share(args):
    """--share-of N (one GPU): the radius graph rank 0 builds in the N-GPU fcc workload — its owned atoms as
    targets over [owned | atoms within the halo width of their bounding box] — timed alone on one GPU, so that
    the per-rank graph time of the multi-GPU line can be looked at kernel by kernel (launch list under ncu)."""
    import torch

    import dynamis_b200 as D
    from dynamis_b200 import synthetic

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K, W = args.steps, max(args.warmup, 3)
    pos_np, cell_np, pbc_np, r = synthetic.fcc_copper(126, seed=1004)
    pos = torch.from_numpy(pos_np).to(dev)
    labels = D.sfc_partition_labels(pos, None, args.share_of, 0)
    own = torch.nonzero(labels == 0).reshape(-1)
    L = float(cell_np[0, 0])
    lo, hi = pos[own].min(dim=0).values, pos[own].max(dim=0).values
    d = ((pos - (lo + hi) / 2 + L / 2) % L - L / 2).abs() - (hi - lo) / 2
    keep = (d <= r + 6.0).all(dim=1)
    keep[own] = False
    allpos = torch.cat([pos[own], pos[torch.nonzero(keep).reshape(-1)]]).contiguous()
    targets = torch.arange(own.numel(), dtype=torch.int64, device=dev)
    cell, pbc = torch.from_numpy(cell_np), torch.from_numpy(pbc_np)
    del pos, labels, keep, d
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(W):
        out = D.radius_graph_pbc_ex(allpos, cell, pbc, r, 0, False, targets)
    E = int(out[2].item())
    del out
    ts = []
    for _ in range(K):
        flush.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = D.radius_graph_pbc_ex(allpos, cell, pbc, r, 0, False, targets)
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
        del out
    ms = float(np.mean(ts))
    print(json.dumps({"metric": "radius_graph_edges_per_s", "value": E / (ms * 1e-3), "unit": "edges/s", "n_gpus": 1, "steps": K,
                      "warmup": W, "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"fcc Cu 8,001,504 atoms, cutoff 6.0 A: rank 0's share of the {args.share_of}-GPU workload on one "
                                             f"GPU, {own.numel()} owned atoms as targets over {allpos.shape[0]} positions",
                                 "edges_per_step": E}}), flush=True)


def run_ours(args):
    import torch

    import dynamis_b200 as D
    from dynamis_b200 import graph as G

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if world > 1:
        import bench_multi

        return bench_multi.run(args, rank, world, dev)

    K, W = args.steps, max(args.warmup, 3)
    pos_np, cell_np, pbc_np, r = liquid(ATOMS_PER_GPU)
    N = pos_np.shape[0]
    pos_pin = torch.from_numpy(pos_np).pin_memory()
    pos = pos_pin.to(dev)
    cell = torch.from_numpy(cell_np)
    pbc = torch.from_numpy(pbc_np)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    have_sfc = hasattr(D, "sfc_partition_labels")

    mid = torch.cuda.Event(enable_timing=True)   # the positions are ready: both halves of the step may start
    gend = torch.cuda.Event(enable_timing=True)  # the radius graph is complete

    # high priority: the partition's short kernels are placed as soon as SM slots free up instead of queueing
    # behind the thousands of blocks of the edge writer
    side = torch.cuda.Stream(device=dev, priority=-1)

    def step(p):
        # The two halves of the step do not depend on each other.  The radius graph is queued first (its call
        # blocks the host once, for the edge count, and returns with the edge writer still running); the Morton
        # partition (short dependent launches) then runs on a second stream beside the edge writer and is joined
        # before the step ends.
        main = torch.cuda.current_stream(dev)
        labels = None
        mid.record()
        out = D.radius_graph_pbc_ex(p, cell, pbc, r, 0, False)
        gend.record()
        if have_sfc:
            side.wait_event(mid)
            with torch.cuda.stream(side):
                labels = D.sfc_partition_labels(p, None, 8, 0)
            main.wait_stream(side)
        return out, labels

    for _ in range(W):
        out, _ = step(pos)
    E = int(out[2].item())
    del out
    torch.cuda.synchronize()

    # ---- device-resident throughput: per-step CUDA events, L2 flushed between steps
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    t_wall0 = time.perf_counter()
    total_ms = 0.0
    graph_ms = 0.0
    for _ in range(K):
        flush.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out, _ = step(pos)
        b.record()
        torch.cuda.synchronize()
        total_ms += a.elapsed_time(b)
        graph_ms += mid.elapsed_time(gend)
        del out
    t_wall1 = time.perf_counter()
    clocks = sampler.stop(t_wall0, t_wall1)
    ms_per_step = total_ms / K
    value = E / (ms_per_step * 1e-3)

    # ---- end to end: positions from pinned host memory, degrees + edge count back to the host
    counts_pin = torch.empty(N, dtype=torch.int32).pin_memory()
    nni_pin = torch.empty(1, dtype=torch.int64).pin_memory()
    pos_in = torch.empty_like(pos)
    for _ in range(2):
        pos_in.copy_(pos_pin, non_blocking=True)
        out, _ = step(pos_in)
        counts_pin.copy_(out[3], non_blocking=True)
        nni_pin.copy_(out[2], non_blocking=True)
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        pos_in.copy_(pos_pin, non_blocking=True)
        out, _ = step(pos_in)
        counts_pin.copy_(out[3], non_blocking=True)
        nni_pin.copy_(out[2], non_blocking=True)
        torch.cuda.synchronize()
        del out
    e2e_s = (time.perf_counter() - t0) / K
    assert int(nni_pin.item()) == E
    e2e = {"value": E / e2e_s, "unit": "edges/s", "ms_per_step": e2e_s * 1e3,
           "h2d_bytes_per_step": int(pos_pin.numel() * 4), "d2h_bytes_per_step": int(N * 4 + 8),
           "note": "positions in from pinned host memory, degrees and edge count out; the 1.47 GB edge list stays on the device, "
                   "as with the API it replaces (CUDA tensors for a CUDA consumer)"}

    # ---- the dominant kernel alone (edge-writing pass), CUDA events on its stream, L2 flushed
    plan = G.plan_radius_graph(pos, cell, pbc, r)
    ei = torch.empty((2, plan.E), dtype=torch.int64, device=dev)
    sh = torch.empty((plan.E, 3), dtype=torch.float32, device=dev)
    for _ in range(3):
        plan.fill_into(ei, sh)
    torch.cuda.synchronize()
    kt = []
    for _ in range(max(K, 10)):
        flush.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        plan.fill_into(ei, sh)
        b.record()
        torch.cuda.synchronize()
        kt.append(a.elapsed_time(b))
    fill_ms = float(np.mean(kt))
    peak, peak_kind = _peaks()
    alg_bytes = 28.0 * plan.E
    achieved = alg_bytes / (fill_ms * 1e-3) / 1e9
    traffic = None
    tp = os.path.join(ROOT, "profiles", "rg_fillmask_traffic.txt")
    if os.path.exists(tp):
        with open(tp) as f:
            tj = json.load(f)
        traffic = tj["dram_bytes_per_edge"] * plan.E
    roofline = {"bound": "hbm", "kernel": "rg_fillmask_kernel<float>", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                "algorithmic_bytes": alg_bytes, "ms_per_launch": fill_ms}
    del ei, sh

    base, _ = cpu_baseline(ATOMS_PER_GPU, steps=1)
    ref_cuda = reference_cuda(pos, cell, pbc, r, E)

    line = {
        "metric": "radius_graph_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "random liquid 1,000,000 atoms, density 0.1 atoms/A^3, cubic periodic box L=215.4 A, fp32, "
                               "cutoff 5.0 A (configs[1]): " + ("Morton partition + " if have_sfc else "") + "radius graph",
                   "edges_per_step": E, "l2": "256 MiB buffer written between timed steps; a step itself writes 1.5 GB"},
        "roofline": roofline, "cpu_baseline": base, "reference_cuda": ref_cuda, "e2e": e2e, "clocks": clocks,
        "gpu_launches": D.launches_per_graph() + (D.launches_per_partition() if have_sfc else 0),
        "halo_exchange_ms_per_step": None,
        # the radius graph alone for comparison with the N > 1 lines (the Morton partition of the step runs beside it on
        # a second stream, so this is close to the whole step)
        "graph_ms_per_step": graph_ms / K, "graph_edges_per_s": E / (graph_ms / K * 1e-3),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="fcc", choices=["fcc", "liquid", "migrate", "exchange"],
                    help="N > 1 only: fcc = 8,001,504-atom fcc Cu cut into N subdomains (strong scaling), liquid = N x 1,000,000 atoms, "
                         "migrate = 4,000,000 drifting atoms with repartition and migration (reports milliseconds per repartition), "
                         "exchange = the pieces of one forward halo push timed apart")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="N > 1 only: one-sided peer stores or NCCL all-to-all")
    ap.add_argument("--share-of", type=int, default=0,
                    help="one GPU: time rank 0's radius graph of the N-GPU fcc workload alone (0 = off)")
    ap.add_argument("--ce-threshold", type=int, default=0, help="N > 1, peer exchange: copy-engine threshold in bytes (0 = SM stores)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.share_of > 1 and args.gpus <= 1:
        run_share(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
