"""Domain partitioners and halo-map construction — host side.

Mirrors the reference's partitioner classes (dynamis_state/include/dynamis_state/partitioner.hpp:6-78,
bound in dynamis_state/src/dynamis_state_bindings.cpp:75-115): ``SFCPartitioner(curve_type)`` and
``SimpleSpatialPartitioner`` with ``partition(state, env[, config])`` and
``build_halo_maps(info, global_state, env, config)`` (fills ``info`` in place).

The compute is in libdynb.so: Morton/"Hilbert" keys, a stable radix sort, the label assignment
(dynb_sfc_partition), bincount / stream compaction (dynb_bincount_i64, dynb_select_eq_i64), and
for the halo maps one cell-scan pass at cutoff + buffer that marks which rank needs which atom
(dynb_rg_halo_mark) followed by CSR assembly (dynb_csr_plan / dynb_csr_fill).  Unlike the
reference, no [N, W] bool matrix and no edge list are materialised.
"""

from __future__ import annotations

import ctypes
import enum
from typing import Optional

import torch

from . import _lib
from .graph import plan_radius_graph, radius_graph_pbc, radius_graph_pbc_ex
from .state import DistEnvironment, MolecularInfo, PartitionMessagePassingInfo, SimulationConfig

PARTITION_MAX_NUM_NEIGHBORS = 1000
HALO_MAX_NUM_NEIGHBORS = 1000

_SCRATCH: dict = {}


def scratch(device: torch.device, name: str, nbytes: int) -> torch.Tensor:
    """Grow-only named device scratch buffers (uint8), one set per (device, stream): work on different streams of
    a device never shares one."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, name)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        _SCRATCH.pop(key, None)
        buf = torch.empty(max(int(nbytes * 1.1) + 256, 256), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


class SFCCurveType(enum.IntEnum):
    Morton = 0
    Hilbert = 1


def launches_per_partition() -> int:
    """Kernels one Morton partition of a million atoms into 8 labels launches (labels only): bounds (1),
    keys (1), 6 digit levels (histogram; its last block advances the split points; once the remaining atoms are few
    the last block settles the split points and the later levels return at once), labels (1).  With the
    curve-order permutation requested the sorted path runs instead: bounds, keys, 8 radix passes x
    (histogram + 2 scan kernels + scatter), assignment."""
    return 1 + 1 + 6 + 1


def sfc_partition_labels(pos: torch.Tensor, weights: Optional[torch.Tensor], W: int, curve_type: int = 0,
                         return_perm: bool = False):
    """Rank label in [0, W) per atom (reference: sfc_partition_cuda, partition/sfc.cpp:9-33)."""
    if not pos.is_cuda:
        raise RuntimeError("pos must be a CUDA tensor")
    if pos.dim() != 2 or pos.size(1) != 3:
        raise RuntimeError(f"pos must have shape [N, 3], got [{pos.size(0)}, {pos.size(1) if pos.dim() > 1 else ''}]")
    if pos.dtype != torch.float32:
        raise RuntimeError(f"pos must be float32, got {pos.dtype}")
    if W < 1:
        raise RuntimeError(f"W must be >= 1, got {W}")
    if curve_type not in (0, 1):
        raise RuntimeError(f"curve_type must be 0 (Morton) or 1 (Hilbert), got {curve_type}")
    pos = pos.contiguous()
    N = pos.size(0)
    dev = pos.device
    if weights is not None:
        if not weights.is_cuda:
            raise RuntimeError("weights must be a CUDA tensor")
        if weights.dim() != 1 or weights.size(0) != N:
            raise RuntimeError(f"weights must have shape [N], got [{weights.size(0)}]")
        weights = weights.to(torch.int64).contiguous()
    L = _lib.lib()
    with _lib.on_device(dev):
        labels = torch.empty((N,), dtype=torch.int64, device=dev)
        perm = torch.empty((N,), dtype=torch.int64, device=dev) if return_perm else None
        if N > 0:
            nbytes = ctypes.c_int64()
            _lib.check(L.dynb_sfc_workspace_bytes(N, ctypes.byref(nbytes)), "sfc_workspace_bytes")
            ws = scratch(dev, "sfc", nbytes.value)
            _lib.check(L.dynb_sfc_partition(pos.data_ptr(), N, weights.data_ptr() if weights is not None else None, int(W),
                                            int(curve_type), labels.data_ptr(), perm.data_ptr() if perm is not None else None,
                                            ws.data_ptr(), ws.numel(), _stream(dev)), "sfc_partition")
    return (labels, perm) if return_perm else labels


def sfc_keys(pos: torch.Tensor, curve_type: int = 0) -> torch.Tensor:
    """Curve keys in atom order, int64 (reference kernels: sfc_kernels.cu:32-109)."""
    pos = pos.contiguous()
    N, dev = pos.size(0), pos.device
    keys = torch.empty((N,), dtype=torch.int64, device=dev)
    if N:
        L = _lib.lib()
        with _lib.on_device(dev):
            nbytes = ctypes.c_int64()
            _lib.check(L.dynb_sfc_workspace_bytes(N, ctypes.byref(nbytes)), "sfc_workspace_bytes")
            ws = scratch(dev, "sfc", nbytes.value)
            _lib.check(L.dynb_sfc_keys(pos.data_ptr(), N, int(curve_type), keys.data_ptr(), ws.data_ptr(), ws.numel(),
                                       _stream(dev)), "sfc_keys")
    return keys


def bincount_labels(labels: torch.Tensor, W: int) -> torch.Tensor:
    dev = labels.device
    L = _lib.lib()
    with _lib.on_device(dev):
        counts = torch.empty((W,), dtype=torch.int64, device=dev)
        bad = scratch(dev, "bad", 256)
        _lib.check(L.dynb_bincount_i64(labels.data_ptr(), labels.numel(), W, counts.data_ptr(), bad.data_ptr(), _stream(dev)),
                   "bincount")
    return counts


def select_eq(values: torch.Tensor, value: int, gather_src: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gather_src[nonzero(values == value)]`` (or the positions themselves), ascending.  One host sync."""
    dev = values.device
    n = values.numel()
    L = _lib.lib()
    with _lib.on_device(dev):
        out = torch.empty((n,), dtype=torch.int64, device=dev)
        cnt = torch.empty((1,), dtype=torch.int64, device=dev)
        nbytes = ctypes.c_int64()
        _lib.check(L.dynb_select_workspace_bytes(n, ctypes.byref(nbytes)), "select_workspace_bytes")
        ws = scratch(dev, "select", nbytes.value)
        _lib.check(L.dynb_select_eq_i64(values.data_ptr(), n, int(value), gather_src.data_ptr() if gather_src is not None else None,
                                        out.data_ptr(), cnt.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)), "select_eq")
        k = int(cnt.item())
    return out[:k]


def _finish_partition(labels: torch.Tensor, state: MolecularInfo, env: DistEnvironment) -> PartitionMessagePassingInfo:
    """partition_indices / atom_counts / matrix from the labels (sfc_partitioner.cpp:164-178)."""
    info = PartitionMessagePassingInfo()
    W, R = int(env.world_size), int(env.global_rank)
    dev = labels.device
    info.partition_id = labels
    info.atom_counts = bincount_labels(labels, W)
    vn = state.atom_vertex_numbers
    vn = vn.to(device=dev, dtype=torch.int64).contiguous() if vn is not None else None
    info.partition_indices = select_eq(labels, R, vn)
    m = torch.zeros((W, W), dtype=torch.int64, device=dev)
    m[R, R] = info.partition_indices.numel()
    info.global_send_recv_matrix = m
    return info


class AbstractPartitioner:
    def build_halo_maps(self, info: PartitionMessagePassingInfo, global_state: MolecularInfo, env: DistEnvironment,
                        config: SimulationConfig) -> None:
        """Send/recv CSR, interior mask and matrix row for rank ``env.global_rank``
        (reference: dynamis_state/src/csrc/build_halo_maps.cpp:20-157)."""
        pos = global_state.atom_positions
        if not pos.is_cuda:
            raise RuntimeError("pos must be a CUDA tensor")
        dev = pos.device
        N, W, R = int(global_state.num_atoms), int(env.world_size), int(env.global_rank)
        ghost_cutoff = float(torch.tensor(config.cutoff + config.ghost_cutoff_buffer, dtype=torch.float32).item())
        pos32 = pos.to(torch.float32).contiguous()
        cell = config.cell.to(torch.float32)
        pbc = config.pbc.to(torch.bool)
        pid = info.partition_id.to(device=dev, dtype=torch.int64).contiguous()
        L = _lib.lib()
        words = (W + 31) // 32
        with _lib.on_device(dev):
            needed = torch.empty((max(N, 1), words), dtype=torch.int32, device=dev)
            has_foreign = torch.empty((max(N, 1),), dtype=torch.uint8, device=dev)
            if N > 0:
                plan = plan_radius_graph(pos32, cell, pbc, ghost_cutoff)
                _lib.check(L.dynb_rg_halo_mark(plan.ws.data_ptr(), plan.dtype_code, pid.data_ptr(), N, W, needed.data_ptr(),
                                               has_foreign.data_ptr(), _stream(dev)), "rg_halo_mark")
            my_indices = select_eq(pid, R)
            n_local = my_indices.numel()
            g2l = torch.empty((max(N, 1),), dtype=torch.int64, device=dev)
            bad = scratch(dev, "bad", 256)
            _lib.check(L.dynb_scatter_iota(my_indices.data_ptr(), n_local, N, g2l.data_ptr(), bad.data_ptr(), _stream(dev)),
                       "scatter_iota")
            nbytes = ctypes.c_int64()
            _lib.check(L.dynb_csr_workspace_bytes(N, W, ctypes.byref(nbytes)), "csr_workspace_bytes")
            ws_s = scratch(dev, "csr_send", nbytes.value)
            ws_r = scratch(dev, "csr_recv", nbytes.value)
            offs = torch.empty((2, W + 1), dtype=torch.int64, device=dev)
            _lib.check(L.dynb_csr_plan(needed.data_ptr(), pid.data_ptr(), N, R, 0, W, offs[0].data_ptr(), ws_s.data_ptr(),
                                       ws_s.numel(), _stream(dev)), "csr_plan(send)")
            _lib.check(L.dynb_csr_plan(needed.data_ptr(), pid.data_ptr(), N, R, 1, W, offs[1].data_ptr(), ws_r.data_ptr(),
                                       ws_r.numel(), _stream(dev)), "csr_plan(recv)")
            offs_h = offs.cpu()
            total_send, total_recv = int(offs_h[0, W]), int(offs_h[1, W])
            send_local = torch.empty((total_send,), dtype=torch.int64, device=dev)
            recv_atom = torch.empty((total_recv,), dtype=torch.int64, device=dev)
            _lib.check(L.dynb_csr_fill(needed.data_ptr(), pid.data_ptr(), N, R, 0, W, g2l.data_ptr(), offs[0].data_ptr(),
                                       send_local.data_ptr(), ws_s.data_ptr(), _stream(dev)), "csr_fill(send)")
            _lib.check(L.dynb_csr_fill(needed.data_ptr(), pid.data_ptr(), N, R, 1, W, None, offs[1].data_ptr(),
                                       recv_atom.data_ptr(), ws_r.data_ptr(), _stream(dev)), "csr_fill(recv)")
            interior = torch.empty((n_local,), dtype=torch.bool, device=dev)
            _lib.check(L.dynb_gather_not_u8(has_foreign.data_ptr(), my_indices.data_ptr(), n_local, interior.data_ptr(),
                                            _stream(dev)), "gather_not_u8")
            info.send_offsets = offs[0].clone()
            info.send_local_indices = send_local
            info.recv_offsets = offs[1].clone()
            info.recv_ghost_indices = torch.arange(n_local, n_local + total_recv, dtype=torch.int64, device=dev)
            info.recv_atom_global = recv_atom
            info.interior_mask = interior
            # build_halo_maps.cpp:150-154
            if info.global_send_recv_matrix is None:
                info.global_send_recv_matrix = torch.zeros((W, W), dtype=torch.int64, device=dev)
            info.global_send_recv_matrix[R] = info.send_offsets[1:] - info.send_offsets[:-1]
            info.global_send_recv_matrix[R, R] = n_local
        info.edge_index_halo = None
        info._edge_index_halo_fn = lambda: radius_graph_pbc(pos32, cell, pbc, ghost_cutoff, HALO_MAX_NUM_NEIGHBORS, False)[0]


class SFCPartitioner(AbstractPartitioner):
    """Cuts the Morton (or "Hilbert") order of the atoms into world_size contiguous runs of equal
    count, or of equal summed ``edge_counts`` (reference: partition/sfc_partitioner.cpp:97-238)."""

    def __init__(self, curve_type: SFCCurveType = SFCCurveType.Morton):
        self.curve_type = SFCCurveType(int(curve_type))

    def partition(self, state: MolecularInfo, env: DistEnvironment, config: Optional[SimulationConfig] = None):
        pos = state.atom_positions
        if not pos.is_cuda:
            raise RuntimeError("SFCPartitioner: atom_positions must be a CUDA tensor (this build has no CPU path)")
        W = int(env.world_size)
        pos32 = pos.to(torch.float32)
        if config is None:
            labels = sfc_partition_labels(pos32, state.edge_counts, W, int(self.curve_type))
            return _finish_partition(labels, state, env)
        # mode 3: weights = in-degree at the cutoff; the graph is kept for downstream use
        cutoff = float(torch.tensor(config.cutoff, dtype=torch.float32).item())
        cell = config.cell.to(torch.float32)
        ei, _, _, counts = radius_graph_pbc_ex(pos32, cell, config.pbc.to(torch.bool), cutoff, PARTITION_MAX_NUM_NEIGHBORS, False)
        labels = sfc_partition_labels(pos32, counts.to(torch.int64), W, int(self.curve_type))
        info = _finish_partition(labels, state, env)
        info.edge_index = ei
        return info


def kdtree_partition_labels(pos: torch.Tensor, weights: Optional[torch.Tensor], W: int, sorted_cuts: bool = False) -> torch.Tensor:
    """Rank label in [0, W) per atom by recursive bisection along the widest axis
    (reference: kdtree_bisect_cuda, partition/kdtree.cpp:9-26).  ``sorted_cuts`` takes the sort-based
    route also for equal-count cuts (same labels)."""
    if not pos.is_cuda:
        raise RuntimeError("pos must be a CUDA tensor")
    if pos.dim() != 2 or pos.size(1) != 3:
        raise RuntimeError(f"pos must have shape [N, 3], got [{pos.size(0)}, {pos.size(1) if pos.dim() > 1 else ''}]")
    if pos.dtype != torch.float32:
        raise RuntimeError(f"pos must be float32, got {pos.dtype}")
    if W < 1:
        raise RuntimeError(f"W must be >= 1, got {W}")
    pos = pos.contiguous()
    N, dev = pos.size(0), pos.device
    if weights is not None:
        if not weights.is_cuda:
            raise RuntimeError("weights must be a CUDA tensor")
        if weights.dim() != 1 or weights.size(0) != N:
            raise RuntimeError(f"weights must have shape [N], got [{weights.size(0)}]")
        weights = weights.to(torch.int64).contiguous()
    L = _lib.lib()
    with _lib.on_device(dev):
        labels = torch.empty((N,), dtype=torch.int64, device=dev)
        if N > 0:
            nbytes = ctypes.c_int64()
            _lib.check(L.dynb_kdtree_workspace_bytes(N, int(W), ctypes.byref(nbytes)), "kdtree_workspace_bytes")
            ws = scratch(dev, "kdtree", nbytes.value)
            _lib.check(L.dynb_kdtree_partition(pos.data_ptr(), N, weights.data_ptr() if weights is not None else None, int(W),
                                               labels.data_ptr(), 1 if sorted_cuts else 0, ws.data_ptr(), ws.numel(), _stream(dev)),
                       "kdtree_partition")
    return labels


class KDTreePartitioner(AbstractPartitioner):
    """Recursive bisection along the widest axis into world_size parts of equal count, or of equal
    summed ``edge_counts``; with a SimulationConfig the weights are the in-degrees at the cutoff and the
    graph is kept (reference: partition/kdtree_partitioner.cpp:52-164)."""

    def partition(self, state: MolecularInfo, env: DistEnvironment, config: Optional[SimulationConfig] = None):
        pos = state.atom_positions
        if not pos.is_cuda:
            raise RuntimeError("KDTreePartitioner: atom_positions must be a CUDA tensor (this build has no CPU path)")
        W = int(env.world_size)
        pos32 = pos.to(torch.float32)
        if config is None:
            labels = kdtree_partition_labels(pos32, state.edge_counts, W)
            return _finish_partition(labels, state, env)
        cutoff = float(torch.tensor(config.cutoff, dtype=torch.float32).item())
        cell = config.cell.to(torch.float32)
        ei, _, _, counts = radius_graph_pbc_ex(pos32, cell, config.pbc.to(torch.bool), cutoff, PARTITION_MAX_NUM_NEIGHBORS, False)
        labels = kdtree_partition_labels(pos32, counts.to(torch.int64), W)
        info = _finish_partition(labels, state, env)
        info.edge_index = ei
        return info


class SimpleSpatialPartitioner(AbstractPartitioner):
    """Contiguous index split: rank r owns atoms [r*(N//W), (r+1)*(N//W)), the last rank the
    remainder (reference: partition/simple_spatial_partitioner.cpp:6-47)."""

    def partition(self, state: MolecularInfo, env: DistEnvironment):
        dev = state.atom_positions.device
        N, W, R = int(state.num_atoms), int(env.world_size), int(env.global_rank)
        per = N // W
        info = PartitionMessagePassingInfo()
        ar = torch.arange(N, dtype=torch.int64, device=dev)
        info.partition_id = torch.clamp(torch.div(ar, per, rounding_mode="trunc"), 0, W - 1) if per > 0 else \
            torch.full((N,), W - 1, dtype=torch.int64, device=dev)
        start = R * per
        end = N if R == W - 1 else start + per
        info.partition_indices = state.atom_vertex_numbers[start:end].contiguous()
        m = torch.zeros((W, W), dtype=torch.int64, device=dev)
        m[R, R] = end - start
        info.global_send_recv_matrix = m
        info.atom_counts = torch.bincount(info.partition_id, minlength=W)
        return info
