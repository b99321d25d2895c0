"""Periodic radius graph — host side of the reference's ``dynamis_state`` graph API.

Same names, argument meaning and error behaviour as the reference's pybind entry points
(dynamis_state/src/dynamis_state_bindings.cpp:153-163, 241-254; validation text from
dynamis_state/src/csrc/graph/radius_graph.cpp:7-127) and its Python wrapper
(dynamis_state/src/dynamis_state/radius_graph_pbc_cuda.py:13-110).  The work is done by the
CUDA kernels behind ``dynb_rg_plan`` / ``dynb_rg_fill``; PyTorch only owns the memory and the
stream.

One extension: positions may be float64 (the reference rejects them); distances are then
evaluated in float64.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from . import _lib

_STATE: dict = {}


def _dev_state(device: torch.device) -> dict:
    """Plan workspace and pinned header of one (device, stream): calls on different streams of a device get
    workspaces of their own and so cannot race on one; calls on one stream are ordered by the stream."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (device.type, index, torch.cuda.current_stream(torch.device("cuda", index)).cuda_stream)
    st = _STATE.get(key)
    if st is None:
        pinned = torch.empty(64, dtype=torch.uint8).pin_memory()
        st = {"ws": None, "hdr_t": pinned, "hdr": _lib.RgHeader.from_address(pinned.data_ptr()), "geo": {}}
        _STATE[key] = st
    return st


def _workspace(st: dict, nbytes: int, device: torch.device) -> torch.Tensor:
    ws = st["ws"]
    if ws is None or ws.numel() < nbytes:
        st["ws"] = None
        ws = torch.empty(int(nbytes * 1.1) + 4096, dtype=torch.uint8, device=device)
        st["ws"] = ws
    return ws


def _validate(pos, cell, pbc, radius, max_num_neighbors, target_indices):
    if not isinstance(pos, torch.Tensor) or not pos.is_cuda:
        raise RuntimeError("pos must be a CUDA tensor")
    if pos.dim() != 2 or pos.size(1) != 3:
        got = ", ".join(str(s) for s in pos.shape)
        raise RuntimeError(f"pos must have shape [N, 3], got [{got}]")
    if pos.dtype not in (torch.float32, torch.float64):
        raise RuntimeError(f"pos must be float32, got {pos.dtype}")
    if cell.dim() != 2 or cell.size(0) != 3 or cell.size(1) != 3:
        got = ", ".join(str(s) for s in cell.shape)
        raise RuntimeError(f"cell must have shape [3, 3], got [{got}]")
    if pbc.dim() != 1 or pbc.size(0) != 3:
        raise RuntimeError(f"pbc must have shape [3], got [{pbc.size(0)}]")
    if not (radius > 0.0):
        raise RuntimeError(f"radius must be positive, got {radius}")
    if max_num_neighbors < 0:
        raise RuntimeError(f"max_num_neighbors must be non-negative, got {max_num_neighbors}")
    if target_indices is not None:
        if target_indices.device != pos.device:
            raise RuntimeError("target_indices must be on the same device as pos")
        if target_indices.dim() != 1:
            raise RuntimeError(f"target_indices must be 1-D, got shape {list(target_indices.shape)}")
        if target_indices.dtype != torch.int64:
            raise RuntimeError(f"target_indices must be int64, got {target_indices.dtype}")


def _empty_result(pos, n_target):
    dev = pos.device
    return (
        torch.empty((2, 0), dtype=torch.int64, device=dev),
        torch.empty((0, 3), dtype=torch.float32, device=dev),
        torch.zeros((1,), dtype=torch.int64, device=dev),
        torch.zeros((n_target,), dtype=torch.int32, device=dev),
    )


class RadiusGraphPlan:
    """Result of the counting phase: degrees are known, the edge buffers are not written yet.

    ``fill()`` may be called more than once (the benchmark times it in isolation); the plan stays
    valid until the next radius-graph call on the same device, which reuses the workspace.
    """

    __slots__ = ("ws", "dtype_code", "E", "M", "counts", "device", "pos_dtype", "max_degree", "grid", "num_groups")

    def fill(self, want_dist_sq: bool = False):
        dev = self.device
        E = self.E
        with _lib.on_device(dev):
            edge_index = torch.empty((2, E), dtype=torch.int64, device=dev)
            shifts = torch.empty((E, 3), dtype=torch.float32, device=dev)
            d2 = torch.empty((E,), dtype=self.pos_dtype, device=dev) if want_dist_sq else None
            self.fill_into(edge_index, shifts, d2)
        return edge_index, shifts, d2

    def fill_into(self, edge_index, shifts, d2=None):
        if self.E == 0:
            return
        stream = torch.cuda.current_stream(self.device)
        _lib.check(_lib.lib().dynb_rg_fill(self.ws.data_ptr(), self.dtype_code, edge_index.data_ptr(), shifts.data_ptr(),
                                           d2.data_ptr() if d2 is not None else None, self.E, stream.cuda_stream),
                   "rg_fill")


    def fill_glue(self, cell: Optional[torch.Tensor], negate_shifts: bool = True, cartesian: bool = True,
                  id_map: Optional[torch.Tensor] = None):
        """Edge list with the shifts in the caller's sign, optionally the Cartesian shifts
        ``unit_shifts @ cell`` (float32) and ids mapped through ``id_map`` (local -> global), all written by
        the edge writer itself."""
        dev = self.device
        E = self.E
        with _lib.on_device(dev):
            edge_index = torch.empty((2, E), dtype=torch.int64, device=dev)
            unit = torch.empty((E, 3), dtype=torch.float32, device=dev)
            cart = torch.empty((E, 3), dtype=torch.float32, device=dev) if cartesian else None
            if E:
                cell_h = None
                if cartesian:
                    cell_h = np.ascontiguousarray(cell.detach().to("cpu").reshape(3, 3).numpy().astype(np.float32))
                if id_map is not None:
                    if id_map.dtype != torch.int64 or not id_map.is_contiguous() or id_map.device != dev:
                        raise RuntimeError("id_map must be a contiguous int64 tensor on the graph's device")
                stream = torch.cuda.current_stream(dev)
                _lib.check(_lib.lib().dynb_rg_fill_glue(self.ws.data_ptr(), self.dtype_code, edge_index.data_ptr(), unit.data_ptr(),
                                                        cart.data_ptr() if cart is not None else None,
                                                        cell_h.ctypes.data if cell_h is not None else None,
                                                        1 if negate_shifts else 0, id_map.data_ptr() if id_map is not None else None,
                                                        E, stream.cuda_stream), "rg_fill_glue")
        return edge_index, unit, cart


def plan_radius_graph(pos, cell, pbc, radius, target_indices=None) -> RadiusGraphPlan:
    """Counting phase (wrap, periodic images, cell binning, degrees, offsets).  Synchronises the
    current stream once to learn the number of edges.  ``pos`` must be non-empty."""
    pos = pos.contiguous()
    N = pos.size(0)
    if target_indices is not None:
        target_indices = target_indices.contiguous()
        Nt = target_indices.size(0)
    else:
        Nt = N
    L = _lib.lib()
    dev = pos.device
    dtype_code = _lib.DYNB_F64 if pos.dtype == torch.float64 else _lib.DYNB_F32
    np_real = np.float64 if pos.dtype == torch.float64 else np.float32
    cell_np = cell.detach().to("cpu").numpy()
    pbc_np = pbc.detach().to("cpu").numpy()

    with _lib.on_device(dev):
        st = _dev_state(dev)
        # the host-side conversions and the capacities of a geometry are kept by value of (cell, pbc, radius, sizes)
        geo_key = (cell_np.tobytes(), str(cell_np.dtype), pbc_np.tobytes(), float(radius), N, dtype_code)
        geo = st["geo"].get(geo_key)
        if geo is None:
            cell_h = np.ascontiguousarray(cell_np.astype(np_real))
            pbc_h = np.ascontiguousarray(pbc_np.astype(bool).astype(np.uint8))
            radius_h = float(np.float32(radius)) if dtype_code == _lib.DYNB_F32 else float(radius)
            src_cap = ctypes.c_int64()
            cell_cap = ctypes.c_int64()
            _lib.check(L.dynb_rg_suggest_capacity(N, cell_h.ctypes.data, pbc_h.ctypes.data, radius_h, dtype_code,
                                                  ctypes.byref(src_cap), ctypes.byref(cell_cap)), "rg_suggest_capacity")
            if len(st["geo"]) > 64:
                st["geo"].clear()
            geo = st["geo"][geo_key] = (cell_h, pbc_h, radius_h, src_cap.value, cell_cap.value)
        cell_h, pbc_h, radius, src_cap, cell_cap = geo
        counts = torch.empty((Nt,), dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev)
        hdr = st["hdr"]
        for attempt in range(3):
            nbytes = ctypes.c_int64()
            _lib.check(L.dynb_rg_workspace_bytes(N, Nt, src_cap, cell_cap, dtype_code, ctypes.byref(nbytes)),
                       "rg_workspace_bytes")
            ws = _workspace(st, nbytes.value, dev)
            _lib.check(L.dynb_rg_plan(pos.data_ptr(), dtype_code, N, cell_h.ctypes.data, pbc_h.ctypes.data, radius,
                                      target_indices.data_ptr() if target_indices is not None else None, Nt,
                                      ws.data_ptr(), ws.numel(), src_cap, cell_cap, counts.data_ptr(),
                                      st["hdr_t"].data_ptr(), stream.cuda_stream), "rg_plan")
            stream.synchronize()
            status = int(hdr.status)
            if status & _lib.RG_SRC_OVERFLOW and attempt < 2:
                src_cap = max(int(hdr.M) + 1024, 2 * src_cap)
                st["geo"][geo_key] = (cell_h, pbc_h, radius, src_cap, cell_cap)  # the next call starts with the larger capacity
                continue
            break
    if status & _lib.RG_BAD_TARGET:
        raise RuntimeError("target_indices contains an index outside [0, N)")
    if status & _lib.RG_NONFINITE:
        raise RuntimeError("pos contains NaN or Inf")
    if status & _lib.RG_SHIFT_RANGE:
        raise RuntimeError("an atom lies too many periodic cells outside the unit cell (limit 511)")
    if status & _lib.RG_SRC_OVERFLOW:
        raise RuntimeError("periodic-image capacity overflow")
    plan = RadiusGraphPlan()
    plan.ws = ws
    plan.dtype_code = dtype_code
    plan.E = int(hdr.E)
    plan.M = int(hdr.M)
    plan.max_degree = int(hdr.max_degree)
    plan.grid = (int(hdr.grid[0]), int(hdr.grid[1]), int(hdr.grid[2]))
    plan.num_groups = int(hdr.num_groups)
    plan.counts = counts
    plan.device = dev
    plan.pos_dtype = pos.dtype
    return plan


def _graph_impl(pos, cell, pbc, radius, target_indices, counts_only, want_dist_sq=False):
    """Shared implementation.  Returns (edge_index, cell_shifts, num_neighbors_image,
    neighbor_counts[, dist_sq])."""
    N = pos.size(0)
    Nt = target_indices.size(0) if target_indices is not None else N
    if N == 0 or Nt == 0:  # reference: radius_graph_kernels.cu:499-509
        out = _empty_result(pos, Nt)
        return out + ((torch.empty(0, dtype=pos.dtype, device=pos.device),) if want_dist_sq else ())
    plan = plan_radius_graph(pos, cell, pbc, radius, target_indices)
    dev = pos.device
    if counts_only or plan.E == 0:  # reference: :802-811, :828-840
        out = (
            torch.empty((2, 0), dtype=torch.int64, device=dev),
            torch.empty((0, 3), dtype=torch.float32, device=dev),
            torch.zeros((1,), dtype=torch.int64, device=dev),
            plan.counts,
        )
        return out + ((torch.empty(0, dtype=pos.dtype, device=dev),) if want_dist_sq else ())
    edge_index, shifts, d2 = plan.fill(want_dist_sq)
    nni = torch.full((1,), plan.E, dtype=torch.int64, device=dev)
    out = (edge_index, shifts, nni, plan.counts)
    return out + ((d2,) if want_dist_sq else ())


def radius_graph_pbc(pos, cell, pbc, radius, max_num_neighbors, enforce_max_strictly):
    """(edge_index [2,E] int64, cell_shifts [E,3] float32, num_neighbors_image [1] int64).

    edge_index row 0 is the neighbour (source), row 1 the centre (target);
    ``pos[src] + cell_shifts @ cell - pos[dst]`` is the edge vector.  ``max_num_neighbors`` and
    ``enforce_max_strictly`` are accepted and ignored, as in the reference
    (radius_graph_kernels.cu:771-775): every neighbour inside the cutoff is returned.
    """
    _validate(pos, cell, pbc, float(radius), int(max_num_neighbors), None)
    ei, cs, nni, _ = _graph_impl(pos, cell, pbc, float(radius), None, False)
    return ei, cs, nni


def radius_graph_pbc_ex(pos, cell, pbc, radius, max_num_neighbors, enforce_max_strictly,
                        target_indices: Optional[torch.Tensor] = None):
    """As radius_graph_pbc, restricted to edges whose centre is in ``target_indices`` (sources stay
    all atoms), plus ``neighbor_counts [N_target] int32`` in the order of ``target_indices``."""
    _validate(pos, cell, pbc, float(radius), int(max_num_neighbors), target_indices)
    return _graph_impl(pos, cell, pbc, float(radius), target_indices, False)


def radius_graph_pbc_counts_ex(pos, cell, pbc, radius, target_indices: Optional[torch.Tensor] = None):
    """Per-target degrees only (no edge buffers, no fill pass)."""
    _validate(pos, cell, pbc, float(radius), 0, target_indices)
    return _graph_impl(pos, cell, pbc, float(radius), target_indices, True)[3]


def radius_graph_pbc_with_dist(pos, cell, pbc, radius, target_indices: Optional[torch.Tensor] = None):
    """Extension: also returns the squared edge lengths the kernel evaluated (dtype of ``pos``)."""
    _validate(pos, cell, pbc, float(radius), 0, target_indices)
    return _graph_impl(pos, cell, pbc, float(radius), target_indices, False, want_dist_sq=True)


def radius_graph_pbc_cuda(data, radius: float, max_num_neighbors_threshold: int,
                          enforce_max_neighbors_strictly: bool = False, pbc: Optional[torch.Tensor] = None):
    """Batch-object wrapper (``data.pos``, ``data.cell [B,3,3]``, ``data.natoms [B]``, ``data.pbc``)."""
    if pbc is None:
        data_pbc = torch.atleast_2d(data.pbc)
        all_true = torch.all(data_pbc, dim=0)
        all_false = torch.all(~data_pbc, dim=0)
        if (~(all_true | all_false)).any():
            raise RuntimeError(
                "Different structures in the batch have different PBC "
                "configurations. This is not currently supported."
            )
        pbc_flags = all_true
    else:
        pbc_flags = pbc.to(torch.bool)

    batch_size = len(data.natoms)
    if batch_size == 1:
        return radius_graph_pbc(data.pos, data.cell[0], pbc_flags, float(radius),
                                int(max_num_neighbors_threshold), enforce_max_neighbors_strictly)
    eis, cos, nns = [], [], []
    natoms = [int(n) for n in data.natoms.tolist()]
    off = 0
    for i, n in enumerate(natoms):
        ei, co, nn = radius_graph_pbc(data.pos[off:off + n], data.cell[i], pbc_flags, float(radius),
                                      int(max_num_neighbors_threshold), enforce_max_neighbors_strictly)
        if ei.size(1) > 0:
            ei = ei + off
        eis.append(ei)
        cos.append(co)
        nns.append(nn)
        off += n
    return torch.cat(eis, dim=1), torch.cat(cos, dim=0), torch.cat(nns, dim=0)


def owned_graph(positions: torch.Tensor, cell: torch.Tensor, pbc: torch.Tensor, cutoff: float, num_local: int,
                negate_shifts: bool = True, cartesian: bool = True):
    """Graph a model builds over [owned | ghost] positions, in one pass.

    The reference models call the radius graph on all exchanged positions and then, in three more passes
    over the edge list, negate the offsets, keep the edges whose destination is an owned atom
    (``edge_index[1] < num_local``) and multiply the unit shifts by the cell
    (dynamis_model/src/dynamis_model/nnp/mace.py:591-608 ``_radius_graph`` / ``_build_owned_graph``,
    uma.py:915-948).  Here the owned destinations are the plan's target subset, and the sign and the
    Cartesian shifts are written by the edge writer.  Returns ``(edge_index [2, E] int64,
    unit_shifts [E, 3] float32, shifts [E, 3] float32 or None)``."""
    pos = positions.contiguous()
    n = pos.size(0)
    num_local = int(num_local)
    if num_local < 0 or num_local > n:
        raise RuntimeError(f"num_local must lie in [0, {n}], got {num_local}")
    _validate(pos, cell.reshape(3, 3), pbc.reshape(-1), cutoff, 0, None)
    dev = pos.device
    if n == 0 or num_local == 0:
        e = torch.empty((2, 0), dtype=torch.int64, device=dev)
        z = torch.empty((0, 3), dtype=torch.float32, device=dev)
        return e, z, (z.clone() if cartesian else None)
    targets = None if num_local == n else torch.arange(num_local, dtype=torch.int64, device=dev)
    plan = plan_radius_graph(pos, cell.reshape(3, 3), pbc.reshape(-1), cutoff, targets)
    return plan.fill_glue(cell, negate_shifts, cartesian)


def launches_per_graph(target_subset: bool = False, fully_periodic: bool = True) -> int:
    """Kernels one radius_graph_pbc call launches on a fully periodic cell: init (header, counters, degrees), wrap
    (which also counts the images into their cells: the grid follows from the cell), 2 scan kernels (source and
    target cell starts together), scatter, finalize, count pass (degrees included), 2 scan kernels (edge offsets),
    two edge-writing launches (the one driven by the hit bits of the count pass and the one that recomputes
    distances; the device decides which of them does the work, the other returns at once; with distances
    requested only the second is launched).  Two more (grid from the data's bounding box, cell histogram) when a
    direction is not periodic or a target subset is given, and two more again (the targets' bounding box, the
    list of groups with targets) with a target subset."""
    n = 11
    if target_subset or not fully_periodic:
        n += 2
    if target_subset:
        n += 2
    return n
