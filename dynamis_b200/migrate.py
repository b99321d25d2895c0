"""Repartition and halo rebuild with the atoms left where they are: no rank ever holds all N atoms.

The reference's ``SimState.sync_and_repartition`` / ``sync_positions_and_rebuild_halo``
(dynamis/src/dynamis/simulatorState.py:136-246) gather every atom to every rank, partition the whole
system on every rank and rebuild the halo maps from a graph of all N atoms.  ``DistributedSimState``
produces the same result — the same owner for every atom, the same owned lists in ascending global id,
the same send / receive CSRs — from per-rank pieces:

  repartition   1. coordinate extrema: six floats min/max-reduced between the ranks
                2. curve keys of the owned atoms against those extrema (same arithmetic as the partition
                   of the gathered system), stable local sort by key
                3. the W - 1 split atoms, i.e. the atoms at the sorted positions where the reference's
                   closed form starts a new label, found by the ranks together: a digit-by-digit descent
                   on (key, global id) in which every rank counts its atoms below 256 candidates per
                   split point and the counts are sum-reduced (8 + at most 4 small all-reduces)
                4. label of every owned atom = number of split atoms <= it (kernel)
                5. atoms that change owner travel in one all-to-all per array; every rank puts what it now
                   owns in ascending global id
  halo maps     6. every rank publishes the box around its atoms (fractional coordinates); atoms within
                   cutoff + buffer of a peer's box go to that peer (a superset of what it needs)
                7. halo marking and CSR assembly run on [owned | received] exactly as build_halo_maps runs
                   them on the whole system: whatever is within reach of an owned atom is in the set

Collectives go through torch.distributed (NCCL on GPUs; staged through the host when the group's backend
is gloo, which is how several ranks share one GPU in tests).
"""

from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .exchange import _pack
from .partition import SFCPartitioner, _stream, scratch
from .state import DistEnvironment, DynamisState, MolecularInfo, PartitionMessagePassingInfo, SimulationConfig


class _Coll:
    """The few collectives used here, on device tensors, for NCCL and (host-staged) gloo groups."""

    def __init__(self, group=None):
        self.group = group
        self.W = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.host = dist.get_backend(group) != "nccl"

    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        if self.host:
            c = t.cpu()
            dist.all_reduce(c, op=op, group=self.group)
            t.copy_(c)
        else:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[W, *t.shape]"""
        src = t.cpu().contiguous() if self.host else t.contiguous()
        out = src.new_empty((self.W,) + tuple(src.shape))
        dist.all_gather_into_tensor(out.view(-1), src.view(-1), group=self.group)
        return out.to(t.device)

    def exchange_counts(self, send_counts: List[int]) -> List[int]:
        s = torch.tensor(send_counts, dtype=torch.int64)
        r = torch.empty_like(s)
        if not self.host:
            dev = torch.device("cuda", torch.cuda.current_device())
            s, r = s.to(dev), r.to(dev)
        dist.all_to_all_single(r, s, group=self.group)
        return [int(v) for v in r.tolist()]

    def all_to_all_rows(self, rows: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        """rows [sum(send_counts), ...] grouped by destination -> rows received, grouped by source."""
        src = rows.cpu().contiguous() if self.host else rows.contiguous()
        out = src.new_empty((sum(recv_counts),) + tuple(src.shape[1:]))
        dist.all_to_all_single(out, src, recv_counts, send_counts, group=self.group)
        return out.to(rows.device)


def _radix_sort_pairs(keys: torch.Tensor, end_bit: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable sort of non-negative int64 keys: (sorted keys, permutation as int64)."""
    n = keys.numel()
    dev = keys.device
    k = keys.clone()
    v = torch.arange(n, dtype=torch.int32, device=dev)
    if n > 1:
        L = _lib.lib()
        nbytes = ctypes.c_int64()
        _lib.check(L.dynb_radix_sort_workspace_bytes(n, ctypes.byref(nbytes)), "radix_sort_workspace_bytes")
        ws = scratch(dev, "migrate_sort", nbytes.value)
        bits = min(64, (max(end_bit, 1) + 7) // 8 * 8)
        with torch.cuda.device(dev):
            _lib.check(L.dynb_radix_sort_pairs(k.data_ptr(), v.data_ptr(), n, 0, bits, ws.data_ptr(), ws.numel(), _stream(dev)),
                       "radix_sort_pairs")
    return k, v.to(torch.int64)


def _gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """x[idx] for a 1-D or 2-D contiguous tensor, through the row-gather kernel."""
    x2 = x.contiguous().view(x.shape[0], -1) if x.dim() > 1 else x.contiguous().view(-1, 1)
    out = torch.empty((idx.numel(),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    _pack(x2, idx.contiguous(), out.view(idx.numel(), -1) if out.dim() > 1 else out.view(-1, 1))
    return out


def split_positions(N: int, W: int) -> List[int]:
    """Sorted position of the first atom of label s + 1, s = 0 .. W - 2 (reference closed form:
    dynamis_state/src/csrc/partition/sfc_kernels.cu:114-137)."""
    base, rem = N // W, N % W
    out = []
    for s in range(1, W):
        out.append(s * (base + 1) if s <= rem else rem * (base + 1) + (s - rem) * base)
    return out


def select_split_atoms(coll, sk: torch.Tensor, sg: torch.Tensor, positions: Optional[List[int]], key_bits: int, id_bits: int,
                       sw: Optional[torch.Tensor] = None, thresholds: Optional[torch.Tensor] = None):
    """(key, id) of the W - 1 split atoms of the union of all ranks' (key, id) lists.  sk / sg: this rank's keys
    and ids in (key, id) order.  Every rank gets the same answer.

    Equal counts: ``positions[s]`` is the global sorted position of split atom s.  Weighted (``sw`` = this rank's
    non-negative int64 weights in the same order, ``thresholds`` int64 [W - 1], non-decreasing): split atom s is
    the first atom, in (key, id) order, whose inclusive prefix weight over all ranks reaches ``thresholds[s]``
    (the reference's rule, dynamis_state/src/csrc/partition/sfc_kernels.cu:165-170, with
    thresholds[s] = ceil((s + 1) * total / W)).  Both are one digit descent: the number — or the weight — of the
    atoms at or below a value is a sorted search into this rank's list, summed over the ranks."""
    dev = sk.device
    weighted = sw is not None
    if weighted:
        want = thresholds.to(device=dev, dtype=torch.int64)
        cw = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), torch.cumsum(sw.to(torch.int64), 0)])
    else:
        want = torch.tensor(positions, dtype=torch.int64, device=dev) + 1       # count of atoms <= split atom
        cw = None
    S = int(want.numel())
    digits = torch.arange(256, dtype=torch.int64, device=dev)

    def descend(sorted_vals, total_bits, base_count, cum, seg_tag=None):
        """Smallest value v (per split) with #(values <= v) >= want - base_count (or their weight, if cum is
        given: cum[i] = weight of the first i values), by 8-bit digits from the top."""
        prefix = torch.zeros(S, dtype=torch.int64, device=dev)
        levels = (total_bits + 7) // 8
        for l in range(levels):
            shift = 8 * (levels - 1 - l)
            low = (1 << shift) - 1
            width = total_bits - shift if l == 0 else 8                                     # the top digit may be narrower
            dd = digits.clamp(max=(1 << width) - 1)
            cand = prefix[:, None] | (dd[None, :] << shift) | low                           # [S, 256] upper ends of the digit ranges
            q = cand if seg_tag is None else (cand | seg_tag[:, None])
            idx = torch.searchsorted(sorted_vals, q.reshape(-1), right=True).reshape(S, 256)
            if cum is None:
                cnt = idx if seg_tag is None else idx - seg_start[:, None]
            else:
                cnt = cum[idx] if seg_tag is None else cum[idx] - cum[seg_start][:, None]
            cnt = coll.all_reduce(cnt.contiguous())
            need = (want - base_count)[:, None]
            d = (cnt < need).sum(dim=1).clamp(max=255)                                     # first digit whose range reaches the rank
            prefix = prefix | (d << shift)
        return prefix

    zero = torch.zeros(S, dtype=torch.int64, device=dev)
    K = descend(sk, key_bits, zero, cw)
    lo = torch.searchsorted(sk, K, right=False)
    hi = torch.searchsorted(sk, K, right=True)
    below = coll.all_reduce((cw[lo] if weighted else lo).clone())                           # atoms (weight) with a smaller key, all ranks
    # ids of the atoms that share the split key, per split point, tagged so that one sorted array serves all
    tag_shift = 40
    if id_bits > tag_shift:
        raise RuntimeError("global atom ids beyond 2^40 are not supported")
    lens = (hi - lo).tolist()
    bounds = list(zip(lo.tolist(), hi.tolist()))
    seg = [sg[a:b] | (s << tag_shift) for s, (a, b) in enumerate(bounds)]
    ties = torch.cat(seg) if seg else sg[:0]
    seg_start = torch.tensor([sum(lens[:s]) for s in range(S)], dtype=torch.int64, device=dev)
    seg_tag = torch.arange(S, dtype=torch.int64, device=dev) << tag_shift
    cum_t = None
    if weighted:
        tw = torch.cat([sw[a:b] for a, b in bounds]) if bounds else sw[:0]
        cum_t = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), torch.cumsum(tw.to(torch.int64), 0)])
    G = descend(ties, id_bits, below, cum_t, seg_tag)
    return K, G


class DistributedSimState:
    """Per-rank simulation state that stays distributed through repartition and halo rebuilds.

    Arguments: this rank's atoms (``global_ids`` ascending, int64; ``positions`` / ``velocities`` float32
    [n, 3]; ``atom_types`` int64 or None), the number of atoms of the whole system, the simulation config
    (cell, pbc, cutoff, ghost_cutoff_buffer) and the rank's DistEnvironment.  ``local_partition_info``
    carries the same fields as the reference's (``partition_indices`` = owned global ids, send / receive
    CSRs, ``recv_atom_global``, ``interior_mask``); ``partition_id`` is not formed (it has one entry per
    atom of the whole system), ``owned_labels`` holds the labels of the atoms this rank held before the
    last repartition instead.
    """

    def __init__(self, global_ids: torch.Tensor, positions: torch.Tensor, velocities: Optional[torch.Tensor],
                 atom_types: Optional[torch.Tensor], num_atoms_total: int, simulation_config: SimulationConfig,
                 distributed_environment: DistEnvironment, curve_type: int = 0, process_group=None):
        self.env = distributed_environment
        self.rank, self.W = int(distributed_environment.global_rank), int(distributed_environment.world_size)
        self.N = int(num_atoms_total)
        self.cfg = simulation_config
        self.curve = int(curve_type)
        self.coll = _Coll(process_group)
        self.device = positions.device
        self.gid = global_ids.to(torch.int64).contiguous()
        self.pos = positions.contiguous()
        self.vel = velocities.contiguous() if velocities is not None else None
        self.types = atom_types.contiguous() if atom_types is not None else None
        self.owned_labels = None
        self.info: Optional[PartitionMessagePassingInfo] = None
        self.last = {}

    # ------------------------------------------------------------------ the reference's accessors
    @property
    def local_partition_info(self) -> PartitionMessagePassingInfo:
        return self.info

    @property
    def state(self) -> DynamisState:
        st = DynamisState()
        loc = MolecularInfo()
        loc.atom_positions, loc.atom_velocities, loc.atom_types, loc.num_atoms = self.pos, self.vel, self.types, self.pos.shape[0]
        st.local_molecular_info, st.local_partition_info, st.sim_config, st.dist_env = loc, self.info, self.cfg, self.env
        return st

    # ------------------------------------------------------------------ steps 1-4
    def new_labels(self, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Label in [0, W) of every atom this rank holds, equal to what the partition of the gathered system
        gives (Morton or "Hilbert" keys, ties by global id): equal counts, or — with ``weights``, one
        non-negative integer per atom this rank holds, e.g. its degree — equal weight (the reference's
        weighted cut, dynamis_state/src/csrc/partition/sfc_kernels.cu:139-173)."""
        if self.N < self.W:
            raise RuntimeError("fewer atoms than ranks")
        L, dev, n = _lib.lib(), self.device, self.pos.shape[0]
        if weights is not None:
            if weights.shape != (n,):
                raise RuntimeError(f"weights must have shape [{n}], got {list(weights.shape)}")
            weights = weights.to(device=dev, dtype=torch.int64)
            if n and int(weights.min()) < 0:
                raise RuntimeError("weights must be non-negative")
        with torch.cuda.device(dev):
            mm = torch.zeros(32, dtype=torch.float32, device=dev)
            _lib.check(L.dynb_sfc_minmax(self.pos.data_ptr(), n, mm.data_ptr(), _stream(dev)), "sfc_minmax")
            lo, hi = mm[:3].clone(), mm[3:6].clone()
            if n == 0:
                lo.fill_(float("inf"))
                hi.fill_(float("-inf"))
            self.coll.all_reduce(lo, dist.ReduceOp.MIN)
            self.coll.all_reduce(hi, dist.ReduceOp.MAX)
            mm[:3], mm[3:6] = lo, hi
            keys = torch.empty(n, dtype=torch.int64, device=dev)
            _lib.check(L.dynb_sfc_keys_from_bounds(self.pos.data_ptr(), n, self.curve, mm.data_ptr(), keys.data_ptr(), _stream(dev)),
                       "sfc_keys_from_bounds")
            key_bits = 63 if self.curve == 0 else 21
            sk, perm = _radix_sort_pairs(keys, key_bits)       # stable: equal keys stay in ascending global id
            sg = self.gid[perm] if n else self.gid
            id_bits = max(1, (self.N - 1).bit_length())
            if weights is None:
                K, G = select_split_atoms(self.coll, sk, sg, split_positions(self.N, self.W), key_bits, id_bits)
            else:
                total = int(self.coll.all_reduce(weights.sum().reshape(1).clone())[0])
                if total == 0:      # the reference labels everything 0 then (sfc_kernels.cu:160-163)
                    return torch.zeros(n, dtype=torch.int64, device=dev)
                thr = torch.tensor([max(1, ((s + 1) * total + self.W - 1) // self.W) for s in range(self.W - 1)], dtype=torch.int64)
                K, G = select_split_atoms(self.coll, sk, sg, None, key_bits, id_bits, sw=weights[perm] if n else weights, thresholds=thr)
            labels = torch.empty(n, dtype=torch.int64, device=dev)
            _lib.check(L.dynb_label_by_splits(keys.data_ptr(), self.gid.data_ptr(), n, K.data_ptr(), G.data_ptr(), self.W - 1,
                                              labels.data_ptr(), _stream(dev)), "label_by_splits")
        return labels

    # ------------------------------------------------------------------ step 5
    def _migrate(self, labels: torch.Tensor) -> None:
        dev, W = self.device, self.W
        order_keys, perm = _radix_sort_pairs(labels, max(1, (W - 1).bit_length()))   # by new owner, ascending id inside
        send_counts = torch.bincount(labels, minlength=W).tolist() if labels.numel() else [0] * W
        recv_counts = self.coll.exchange_counts(send_counts)
        self.last["atoms_leaving"] = int(sum(send_counts) - send_counts[self.rank])

        def move(x):
            if x is None:
                return None
            return self.coll.all_to_all_rows(_gather_rows(x, perm), send_counts, recv_counts)

        gid, pos, vel, types = move(self.gid), move(self.pos), move(self.vel), move(self.types)
        # what arrived is grouped by source rank; owned lists are kept in ascending global id
        _, p2 = _radix_sort_pairs(gid, max(1, (self.N - 1).bit_length()))
        self.gid = _gather_rows(gid, p2)
        self.pos = _gather_rows(pos, p2)
        self.vel = _gather_rows(vel, p2) if vel is not None else None
        self.types = _gather_rows(types, p2) if types is not None else None

    # ------------------------------------------------------------------ steps 6-7
    def rebuild_halo(self) -> PartitionMessagePassingInfo:
        """Halo maps for the current owners and positions (the reference's sync_positions_and_rebuild_halo,
        simulatorState.py:201-246, without gathering the positions)."""
        dev, W, R = self.device, self.W, self.rank
        cfg = self.cfg
        n = self.pos.shape[0]
        cell = cfg.cell.to(device=dev, dtype=torch.float64)
        pbc = [bool(v) for v in cfg.pbc.tolist()]
        reach = float(cfg.cutoff) + float(cfg.ghost_cutoff_buffer)
        inv = torch.linalg.inv(cell)
        # distance between opposite faces along each lattice direction: volume / |a_j x a_k|
        vol = torch.abs(torch.det(cell))
        faces = torch.stack([vol / torch.linalg.norm(torch.linalg.cross(cell[(k + 1) % 3], cell[(k + 2) % 3])) for k in range(3)])
        margin = reach / faces * 1.0001 + 1e-6                                # in fractional units, a little generous
        frac = self.pos.to(torch.float64) @ inv
        if n:
            box = torch.cat([frac.min(dim=0).values, frac.max(dim=0).values])
        else:
            box = torch.tensor([1e30] * 3 + [-1e30] * 3, dtype=torch.float64, device=dev)
        boxes = self.coll.all_gather(box)                                      # [W, 6]
        send_idx, send_counts = [], []
        for p in range(W):
            if p == R or n == 0 or boxes[p, 0] > boxes[p, 3]:
                send_idx.append(torch.empty(0, dtype=torch.int64, device=dev))
                send_counts.append(0)
                continue
            centre, half = (boxes[p, :3] + boxes[p, 3:]) / 2, (boxes[p, 3:] - boxes[p, :3]) / 2
            d = frac - centre
            for k in range(3):
                if pbc[k]:
                    d[:, k] = d[:, k] - torch.round(d[:, k])                    # nearest periodic copy of the box centre
            near = ((d.abs() - half) <= margin).all(dim=1)
            idx = torch.nonzero(near).reshape(-1)
            send_idx.append(idx)
            send_counts.append(int(idx.numel()))
        recv_counts = self.coll.exchange_counts(send_counts)
        sel = torch.cat(send_idx)
        cand_gid = self.coll.all_to_all_rows(_gather_rows(self.gid, sel), send_counts, recv_counts)
        cand_pos = self.coll.all_to_all_rows(_gather_rows(self.pos, sel), send_counts, recv_counts)
        self.last["halo_candidates"] = int(cand_gid.numel())

        set_pos = torch.cat([self.pos, cand_pos])
        set_gid = torch.cat([self.gid, cand_gid])
        owner = torch.cat([torch.full((n,), R, dtype=torch.int64, device=dev)] +
                          [torch.full((c,), p, dtype=torch.int64, device=dev) for p, c in enumerate(recv_counts)])
        mol = MolecularInfo()
        mol.num_atoms, mol.atom_positions = int(set_pos.shape[0]), set_pos
        mol.atom_vertex_numbers = torch.arange(set_pos.shape[0], dtype=torch.int64, device=dev)
        info = PartitionMessagePassingInfo()
        info.partition_id = owner
        info.partition_indices = torch.arange(n, dtype=torch.int64, device=dev)
        SFCPartitioner().build_halo_maps(info, mol, self.env, cfg)
        info.recv_atom_global = set_gid[info.recv_atom_global]                 # set index -> global id
        info.partition_indices = self.gid
        info.partition_id = None
        info.atom_counts = None
        info._edge_index_halo_fn = None
        self.info = info
        return info

    def repartition(self, weights: Optional[torch.Tensor] = None) -> PartitionMessagePassingInfo:
        """The reference's sync_and_repartition (simulatorState.py:136-199) on distributed state; ``weights``
        (per atom this rank holds) selects the weighted cut."""
        labels = self.new_labels(weights)
        self.owned_labels = labels
        self._migrate(labels)
        return self.rebuild_halo()
