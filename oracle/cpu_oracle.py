"""TEST INFRASTRUCTURE ONLY — CPU oracle for the graph / partition / halo path.

A restatement of the reference's algorithms on the CPU: the radius graph in C
(``liborc.so``, see rg_oracle.c), everything else in numpy.  Each function
cites the reference file:line it follows (paths inside the reference project).

Pinning status
  * radius graph, float32: pinned against the reference's own CUDA build by the
    GPU parity tests and by the committed fixtures under tests/golden/ that
    were produced by that build.
  * radius graph, float64: parity unpinned (the reference rejects float64).
  * SFC keys / labels, halo maps, extract_halo_info: pinned by the same golden
    fixtures and by the closed-form invariants the reference's tests assert.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import
this module.  The product (dynamis_b200) never does.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class _OrcGraph(ctypes.Structure):
    _fields_ = [
        ("E", ctypes.c_int64),
        ("Nt", ctypes.c_int64),
        ("M", ctypes.c_int64),
        ("src", ctypes.POINTER(ctypes.c_int64)),
        ("dst", ctypes.POINTER(ctypes.c_int64)),
        ("shift", ctypes.POINTER(ctypes.c_int32)),
        ("counts", ctypes.POINTER(ctypes.c_int32)),
        ("d2", ctypes.POINTER(ctypes.c_double)),
    ]


def build(force: bool = False) -> str:
    """Compile liborc.so with the Makefile next to this file (gcc, a few seconds)."""
    so = os.path.join(_HERE, "liborc.so")
    srcs = [os.path.join(_HERE, f) for f in ("rg_oracle.c", "rg_oracle_impl.h", "integrator_oracle.c", "Makefile")]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.run(["make", "-C", _HERE, "-s", "liborc.so"], check=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liborc.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        for name, real in (("orc_radius_graph_f32", ctypes.c_float), ("orc_radius_graph_f64", ctypes.c_double)):
            fn = getattr(L, name)
            fn.restype = ctypes.POINTER(_OrcGraph)
            fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, real,
                           ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.orc_graph_free.argtypes = [ctypes.POINTER(_OrcGraph)]
        L.orc_graph_free.restype = None
        L.orc_max_threads.restype = ctypes.c_int
        L.orc_geometry_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.orc_geometry_f32.restype = None
        L.orc_edge_keep_mask_f32.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_float, ctypes.c_int64, ctypes.c_void_p]
        L.orc_edge_keep_mask_f32.restype = None
        L.orc_integrator_step.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 5 + [ctypes.c_int64] + [ctypes.c_float] * 3
        L.orc_integrator_step.restype = None
        L.orc_drift_flag.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_float, ctypes.c_float]
        L.orc_drift_flag.restype = ctypes.c_int
        _LIB = L
    return _LIB


def integrator_step(kind, pos, vel, frc, mass, noise, dt, gamma=0.0, kT=0.0):
    """In-place integrator step on float32 numpy arrays (integrator_oracle.c).  kind: 0 Euler, 1/2 Verlet
    half-steps, 3/4 Langevin half-steps; ``pos`` may be None for 2 and 4, ``noise`` for 0-2."""
    p = (lambda a: a.ctypes.data if a is not None else None)
    for a in (pos, vel, frc, mass, noise):
        assert a is None or (a.dtype == np.float32 and a.flags.c_contiguous)
    lib().orc_integrator_step(int(kind), p(pos), p(vel), p(frc), p(mass), p(noise), vel.shape[0], dt, gamma, kT)


def drift_flag(cur, ref, vel, prev_vel, dt, threshold) -> int:
    """2-bit drift word (simulatorState.py:257-293); prev_vel is overwritten with vel."""
    for a in (cur, ref, vel, prev_vel):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    return int(lib().orc_drift_flag(cur.ctypes.data, ref.ctypes.data, vel.ctypes.data, prev_vel.ctypes.data, cur.shape[0], dt, threshold))


def max_threads() -> int:
    return int(lib().orc_max_threads())


# --------------------------------------------------------------------------- radius graph

def radius_graph(pos, cell, pbc, radius, targets=None, nthreads: int = 0):
    """Directed periodic radius graph (reference: radius_graph_kernels.cu:479-934).

    ``pos`` float32 or float64 [N,3]; returns a dict with ``src``/``dst`` int64 [E]
    (edge_index rows 0/1), ``shift`` int32 [E,3], ``counts`` int32 [N_t] in the
    order of ``targets`` (or atom order), ``d2`` float64 [E], ``E`` and ``M``.
    """
    pos = np.ascontiguousarray(pos)
    if pos.dtype not in (np.float32, np.float64):
        raise TypeError("pos must be float32 or float64")
    real = pos.dtype
    cell = np.ascontiguousarray(cell, dtype=real)
    pbc8 = np.ascontiguousarray(np.asarray(pbc, dtype=bool).astype(np.uint8))
    N = pos.shape[0]
    if targets is not None:
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        tptr, nt = targets.ctypes.data, targets.shape[0]
    else:
        tptr, nt = None, N
    fn = lib().orc_radius_graph_f32 if real == np.float32 else lib().orc_radius_graph_f64
    rad = float(np.float32(radius)) if real == np.float32 else float(radius)
    g = fn(pos.ctypes.data if N else None, N, cell.ctypes.data, pbc8.ctypes.data, rad, tptr, nt, nthreads)
    try:
        E = int(g.contents.E)
        out = {
            "E": E,
            "M": int(g.contents.M),
            "src": np.ctypeslib.as_array(g.contents.src, shape=(E,)).copy() if E else np.zeros(0, np.int64),
            "dst": np.ctypeslib.as_array(g.contents.dst, shape=(E,)).copy() if E else np.zeros(0, np.int64),
            "shift": np.ctypeslib.as_array(g.contents.shift, shape=(E, 3)).copy() if E else np.zeros((0, 3), np.int32),
            "d2": np.ctypeslib.as_array(g.contents.d2, shape=(E,)).copy() if E else np.zeros(0, np.float64),
            "counts": np.ctypeslib.as_array(g.contents.counts, shape=(max(nt, 1),))[:nt].copy(),
        }
    finally:
        lib().orc_graph_free(g)
    return out


def geometry(cell, pbc, radius):
    """rep[3], cutoff_frac[3], inverse[3,3] as the reference's host code computes them
    (radius_graph_kernels.cu:516-587), float32."""
    cell = np.ascontiguousarray(cell, dtype=np.float32)
    pbc8 = np.ascontiguousarray(np.asarray(pbc, dtype=bool).astype(np.uint8))
    rep = np.zeros(3, np.int32)
    cf = np.zeros(3, np.float32)
    inv = np.zeros(9, np.float32)
    lib().orc_geometry_f32(cell.ctypes.data, pbc8.ctypes.data, float(np.float32(radius)),
                           rep.ctypes.data, cf.ctypes.data, inv.ctypes.data)
    return rep, cf, inv.reshape(3, 3)


def canonical_edges(src, dst, shift):
    """Canonical form of an edge set: rows (dst, src, sx, sy, sz) int64, sorted
    lexicographically.  Wider fields than the 14-bit packing of the reference's test
    helper (dynamis_state/tests/test_radius_graph_pbc_cuda.py:52-72), which overflows
    above 16k atoms."""
    src = np.asarray(src, dtype=np.int64).ravel()
    dst = np.asarray(dst, dtype=np.int64).ravel()
    sh = np.rint(np.asarray(shift, dtype=np.float64)).astype(np.int64).reshape(-1, 3)
    rows = np.stack([dst, src, sh[:, 0], sh[:, 1], sh[:, 2]], axis=1)
    if rows.shape[0] == 0:
        return rows
    order = np.lexsort((rows[:, 4], rows[:, 3], rows[:, 2], rows[:, 1], rows[:, 0]))
    return rows[order]


def edge_set_digest(src, dst, shift) -> tuple[int, int]:
    """Order-independent digest (count, sum of per-edge 64-bit hashes mod 2^64)."""
    src = np.asarray(src, dtype=np.int64).astype(np.uint64)
    dst = np.asarray(dst, dtype=np.int64).astype(np.uint64)
    sh = (np.rint(np.asarray(shift, dtype=np.float64)).astype(np.int64) + 512).astype(np.uint64).reshape(-1, 3)
    with np.errstate(over="ignore"):
        h = src * np.uint64(0x9E3779B97F4A7C15) + dst * np.uint64(0xC2B2AE3D27D4EB4F)
        h ^= (sh[:, 0] << np.uint64(40)) | (sh[:, 1] << np.uint64(20)) | sh[:, 2]
        h *= np.uint64(0xD6E8FEB86659FD93)
        h ^= h >> np.uint64(32)
        total = int(np.sum(h, dtype=np.uint64))
    return int(src.shape[0]), total


def filter_edges_to_radius(edges, shifts, pos, cell, radius):
    """Order-preserving edge filter (dist_graph_ops_kernels.cu:16-43, 62-102)."""
    edges = np.ascontiguousarray(edges, dtype=np.int64)
    E = edges.shape[1]
    if E == 0:
        return edges, shifts
    src = np.ascontiguousarray(edges[0])
    dst = np.ascontiguousarray(edges[1])
    sh = np.ascontiguousarray(shifts, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.float32)
    cell = np.ascontiguousarray(cell, dtype=np.float32)
    keep = np.zeros(E, np.uint8)
    r2 = float(np.float32(float(radius) * float(radius)))
    lib().orc_edge_keep_mask_f32(src.ctypes.data, dst.ctypes.data, sh.ctypes.data, pos.ctypes.data,
                                 cell.ctypes.data, r2, E, keep.ctypes.data)
    idx = np.nonzero(keep)[0]
    return edges[:, idx], np.asarray(shifts)[idx]


# --------------------------------------------------------------------------- SFC partition

def _spread_bits_21(v):
    x = v.astype(np.uint64) & np.uint64(0x1FFFFF)
    x = (x | (x << np.uint64(32))) & np.uint64(0x1F00000000FFFF)
    x = (x | (x << np.uint64(16))) & np.uint64(0x1F0000FF0000FF)
    x = (x | (x << np.uint64(8))) & np.uint64(0x100F00F00F00F00F)
    x = (x | (x << np.uint64(4))) & np.uint64(0x10C30C30C30C30C3)
    x = (x | (x << np.uint64(2))) & np.uint64(0x1249249249249249)
    return x


def _normalised(pos):
    pos = np.asarray(pos, dtype=np.float32)
    pmin = pos.min(axis=0)
    prange = pos.max(axis=0) - pmin
    prange = np.where(prange > 0, prange, np.float32(1.0)).astype(np.float32)
    return ((pos - pmin) / prange).astype(np.float32)


def sfc_keys(pos, curve_type: int = 0):
    """Morton (0) or the reference's 7-bit "Hilbert" (1) keys, int64 [N]
    (dynamis_state/src/csrc/partition/sfc_kernels.cu:19-56 and :62-109)."""
    n = _normalised(pos)
    if curve_type == 0:
        gm = np.float32((1 << 21) - 1)
        q = np.minimum((n * gm).astype(np.float32).astype(np.int64), (1 << 21) - 1).astype(np.uint64)
        key = _spread_bits_21(q[:, 0]) | (_spread_bits_21(q[:, 1]) << np.uint64(1)) | (_spread_bits_21(q[:, 2]) << np.uint64(2))
        return key.astype(np.int64)
    gm = np.float32(127)
    q = np.clip((n * gm).astype(np.float32).astype(np.int64), 0, 127)
    x, y, z = q[:, 0], q[:, 1], q[:, 2]
    res = np.zeros(q.shape[0], np.int64)
    for b in range(7):
        xb, yb, zb = (x >> b) & 1, (y >> b) & 1, (z >> b) & 1
        if b == 0:
            nxb, nyb, nzb = xb, yb, zb
        else:
            nxb = np.where(xb == 1, zb, xb)
            nyb = np.where(xb == 1, yb, np.where(yb == 1, zb, yb))
            nzb = np.where(xb == 1, yb, np.where(yb == 1, xb, np.where(zb == 1, yb, zb)))
        res |= (nxb << (3 * b)) | (nyb << (3 * b + 1)) | (nzb << (3 * b + 2))
    return res


def sfc_partition(pos, weights, W: int, curve_type: int = 0):
    """Partition labels int64 [N] (sfc_kernels.cu:114-251).  Ties between equal keys are
    broken by atom index (a stable sort); the reference's sort leaves them unspecified."""
    N = np.asarray(pos).shape[0]
    if W == 1:
        return np.zeros(N, np.int64)
    keys = sfc_keys(pos, curve_type)
    perm = np.argsort(keys, kind="stable")
    labels = np.empty(N, np.int64)
    i = np.arange(N, dtype=np.int64)
    if weights is not None:
        cs = np.cumsum(np.asarray(weights).astype(np.int64)[perm])
        total = int(cs[-1]) if N else 0
        p = (cs * W) // total if total > 0 else np.zeros(N, np.int64)
        p = np.clip(p, 0, W - 1)
    else:
        base, rem = N // W, N % W
        thr = rem * (base + 1)
        with np.errstate(divide="ignore", invalid="ignore"):
            hi = rem + ((i - thr) // base if base > 0 else np.zeros(N, np.int64))
        p = np.where(i < thr, i // (base + 1), hi)
        p = np.minimum(p, W - 1)
    labels[perm] = p
    return labels


# --------------------------------------------------------------------------- halo maps

def _csr(counts_per_rank, W):
    off = np.zeros(W + 1, np.int64)
    off[1:] = np.cumsum(counts_per_rank)
    return off


def build_halo_maps(src, dst, partition_id, R: int, W: int):
    """Send/recv CSR and interior mask from the full graph at cutoff + buffer
    (dynamis_state/src/csrc/build_halo_maps.cpp:50-154)."""
    pid = np.asarray(partition_id, dtype=np.int64)
    N = pid.shape[0]
    src = np.asarray(src, dtype=np.int64)
    dst = np.asarray(dst, dtype=np.int64)
    needed = np.zeros((N, W), bool)
    needed[np.arange(N), pid] = True
    needed[src, pid[dst]] = True
    my_idx = np.nonzero(pid == R)[0]
    n_local = my_idx.shape[0]
    mine = needed[my_idx].copy()
    mine[:, R] = False
    rows, ranks = np.nonzero(mine)
    order = np.argsort(ranks, kind="stable")
    send_local = rows[order].astype(np.int64)
    send_off = _csr(np.bincount(ranks, minlength=W), W)
    i_need = needed[:, R].copy()
    i_need[pid == R] = False
    recv_global = np.nonzero(i_need)[0]
    rr = pid[recv_global]
    rorder = np.argsort(rr, kind="stable")
    recv_off = _csr(np.bincount(rr, minlength=W), W)
    recv_atom = recv_global[rorder].astype(np.int64)
    dmine = pid[dst] == R
    ghost_src = pid[src[dmine]] != R
    has_ghost = np.zeros(N, bool)
    has_ghost[dst[dmine][ghost_src]] = True
    interior = ~has_ghost[my_idx]
    matrix_row = send_off[1:] - send_off[:-1]
    matrix_row[R] = n_local
    return {
        "send_offsets": send_off,
        "send_local_indices": send_local,
        "recv_offsets": recv_off,
        "recv_ghost_indices": np.arange(n_local, n_local + recv_atom.shape[0], dtype=np.int64),
        "recv_atom_global": recv_atom,
        "interior_mask": interior,
        "matrix_row": matrix_row.astype(np.int64),
        "num_local": n_local,
    }


def extract_halo_info(edges, pid_outer, my_outer_atoms, my_rank: int, W: int, N: int):
    """The same CSRs from one rank's edge list (dst in my atoms), via the graph's symmetry
    (dynamis_state/src/csrc/graph/dist_graph_ops_kernels.cu:104-188)."""
    edges = np.asarray(edges, dtype=np.int64)
    pid = np.asarray(pid_outer, dtype=np.int64)
    mine = np.asarray(my_outer_atoms, dtype=np.int64)
    n_local = mine.shape[0]
    src, dst = edges[0], edges[1]
    peer = pid[src]
    b = peer != my_rank
    b_src, b_dst, b_peer = src[b], dst[b], peer[b]
    g2l = np.full(N, -1, np.int64)
    g2l[mine] = np.arange(n_local)
    rk = np.unique(b_peer * N + b_src)
    recv_peer, recv_atom = rk // N, rk % N
    recv_off = _csr(np.bincount(recv_peer, minlength=W), W)
    sk = np.unique(b_peer * N + b_dst)
    send_peer, send_atom = sk // N, sk % N
    send_off = _csr(np.bincount(send_peer, minlength=W), W)
    has_remote = np.zeros(N, bool)
    has_remote[b_dst] = True
    return (send_off, g2l[send_atom], recv_off,
            np.arange(n_local, n_local + recv_atom.shape[0], dtype=np.int64),
            ~has_remote[mine], recv_atom.astype(np.int64))


# --------------------------------------------------------------------------- halo exchange

def exchange_forward(features, send_offsets, send_local_indices, recv_offsets):
    """All ranks at once.  ``features[r]`` is [n_local_r, F]; returns per rank the
    concatenated [local | ghosts grouped by owner rank] tensor
    (dynamis_model/src/dynamis_model/comm/exchanger.py:206-240)."""
    W = len(features)
    out = []
    for r in range(W):
        ghosts = []
        for p in range(W):
            so, sl = send_offsets[p], send_local_indices[p]
            rows = sl[so[r]:so[r + 1]]
            assert rows.shape[0] == recv_offsets[r][p + 1] - recv_offsets[r][p]
            ghosts.append(features[p][rows])
        out.append(np.concatenate([features[r]] + ghosts, axis=0))
    return out


def exchange_backward(grads, num_local, send_offsets, send_local_indices, recv_offsets):
    """Reverse halo: ghost-row gradients return to their owners and are added in
    (exchanger.py:277-314).  ``grads[r]`` is [n_local_r + n_ghost_r, F]; accumulation in
    float64 so the result is the exact sum rounded once."""
    W = len(grads)
    out = []
    for r in range(W):
        acc = grads[r][:num_local[r]].astype(np.float64).copy()
        for p in range(W):
            rows = send_local_indices[r][send_offsets[r][p]:send_offsets[r][p + 1]]
            g0 = num_local[p] + recv_offsets[p][r]
            np.add.at(acc, rows, grads[p][g0:g0 + rows.shape[0]].astype(np.float64))
        out.append(acc)
    return out


def _sortable_u32(x):
    """Order-preserving map float32 -> uint32 (kdtree_kernels.cu:9-14)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return np.where(b >> 31, ~b, b | np.uint32(0x80000000)).astype(np.uint32)


def kdtree_partition(pos, weights, W):
    """Labels of the recursive bisection along the widest axis, level by level as the reference's CUDA
    driver does it (dynamis_state/src/csrc/partition/kdtree_kernels.cu:264-467; the same rule as the
    host recursion, kdtree_partitioner.cpp:10-50): per segment the axis of largest extent (first on
    ties), a stable sort by (segment, coordinate), the split at size // 2 (equal counts) or at the
    first position whose inclusive prefix weight reaches half of the segment's weight, clamped to
    [1, size - 1].  Weights are summed as exact integers (the reference's float32 cumulative sum is
    identical while all sums stay below 2**24)."""
    pos = np.ascontiguousarray(pos, dtype=np.float32)
    n = pos.shape[0]
    if W == 1 or n == 0:
        return np.zeros(n, dtype=np.int64)
    levels = int(np.ceil(np.log2(W)))
    parts = [int(W)]
    seg = np.zeros(n, dtype=np.int64)
    w = None if weights is None else np.asarray(weights, dtype=np.int64)
    for _ in range(levels):
        S = len(parts)
        child_l, child_r, nxt = [], [], []
        for p in parts:
            if p <= 1:
                child_l.append(len(nxt)); child_r.append(len(nxt)); nxt.append(p)
            else:
                child_l.append(len(nxt)); nxt.append(p // 2)
                child_r.append(len(nxt)); nxt.append(p - p // 2)
        coord = np.empty(n, dtype=np.float32)
        for s in range(S):
            m = seg == s
            if not m.any():
                continue
            ext = pos[m].max(axis=0) - pos[m].min(axis=0)          # float32 subtraction, as the kernel
            axis, best = 0, np.float32(-1.0)
            for d in range(3):
                if ext[d] > best:
                    best, axis = ext[d], d
            coord[m] = pos[m, axis]
        key = (seg.astype(np.uint64) << np.uint64(32)) | _sortable_u32(coord).astype(np.uint64)
        order = np.argsort(key, kind="stable")
        new_seg = np.empty(n, dtype=np.int64)
        start = 0
        for s in range(S):
            sz = int((seg == s).sum())
            idx = order[start:start + sz]
            if parts[s] <= 1 or sz <= 1:
                mid = sz
            elif w is None:
                mid = min(max(sz // 2, 1), sz - 1)
            else:
                cs = np.cumsum(w[idx])
                total = int(cs[-1])
                lo = int(np.searchsorted(2 * cs >= total, True))   # first position with 2 * cumsum >= total
                mid = min(max(lo, 1), sz - 1)
            new_seg[idx[:mid]] = child_l[s]
            new_seg[idx[mid:]] = child_r[s]
            start += sz
        seg, parts = new_seg, nxt
    base = np.concatenate([[0], np.cumsum(parts)[:-1]]).astype(np.int64)
    return base[seg]
