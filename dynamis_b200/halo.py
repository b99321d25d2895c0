"""Distributed-graph helper ops — host side of ``filter_edges_to_radius`` and ``extract_halo_info``.

Same signatures, validation text and result order as the reference's entry points
(dynamis_state/src/csrc/graph/dist_graph_ops.cpp:5-60, bound at
dynamis_state/src/dynamis_state_bindings.cpp:249-263).
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .partition import _stream, scratch


def filter_edges_to_radius(edges: torch.Tensor, cell_shifts: torch.Tensor, pos: torch.Tensor, cell: torch.Tensor,
                           radius: float):
    """Keeps edge e iff ``|pos[src] + shift @ cell - pos[dst]|^2 <= radius^2`` (float32); order preserving.
    Returns (edges [2,E'], cell_shifts [E',3] in the input dtype)."""
    if not edges.is_cuda:
        raise RuntimeError("edges must be a CUDA tensor")
    if edges.dim() != 2 or edges.size(0) != 2:
        raise RuntimeError(f"edges must have shape [2, E], got {list(edges.shape)}")
    if edges.dtype != torch.int64:
        raise RuntimeError(f"edges must be int64, got {edges.dtype}")
    E = edges.size(1)
    if cell_shifts.dim() != 2 or cell_shifts.size(1) != 3:
        raise RuntimeError(f"cell_shifts must have shape [E, 3], got {list(cell_shifts.shape)}")
    if cell_shifts.size(0) != E:
        raise RuntimeError(f"cell_shifts rows ({cell_shifts.size(0)}) must equal number of edges E ({E})")
    if not pos.is_cuda:
        raise RuntimeError("pos must be a CUDA tensor")
    if pos.dim() != 2 or pos.size(1) != 3:
        raise RuntimeError(f"pos must have shape [N, 3], got {list(pos.shape)}")
    if pos.dtype != torch.float32:
        raise RuntimeError(f"pos must be float32, got {pos.dtype}")
    if cell.dim() != 2 or cell.size(0) != 3 or cell.size(1) != 3:
        raise RuntimeError(f"cell must have shape [3, 3], got {list(cell.shape)}")
    if not (radius > 0.0):
        raise RuntimeError(f"radius must be positive, got {radius}")
    if E == 0:
        return edges, cell_shifts
    edges = edges.contiguous()
    cell_shifts = cell_shifts.contiguous()
    pos = pos.contiguous()
    dev = pos.device
    cell_h = np.ascontiguousarray(cell.detach().to("cpu", torch.float32).numpy())
    shifts_f = cell_shifts if cell_shifts.dtype == torch.float32 else cell_shifts.to(torch.float32)
    L = _lib.lib()
    with torch.cuda.device(dev):
        nbytes = ctypes.c_int64()
        _lib.check(L.dynb_select_workspace_bytes(2 * E, ctypes.byref(nbytes)), "select_workspace_bytes")
        ws = scratch(dev, "filter", nbytes.value)
        cnt = torch.empty((1,), dtype=torch.int64, device=dev)
        _lib.check(L.dynb_filter_edges_plan(edges.data_ptr(), shifts_f.data_ptr(), pos.data_ptr(), cell_h.ctypes.data,
                                            float(radius), E, cnt.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)),
                   "filter_edges_plan")
        E_out = int(cnt.item())
        edges_out = torch.empty((2, E_out), dtype=torch.int64, device=dev)
        shifts_out = torch.empty((E_out, 3), dtype=cell_shifts.dtype, device=dev)
        _lib.check(L.dynb_filter_edges_fill(edges.data_ptr(), cell_shifts.data_ptr(), 3 * cell_shifts.element_size(), E, E_out,
                                            edges_out.data_ptr(), shifts_out.data_ptr(), ws.data_ptr(), _stream(dev)),
                   "filter_edges_fill")
    return edges_out, shifts_out


def extract_halo_info(edges: torch.Tensor, pid_outer: torch.Tensor, my_outer_atoms: torch.Tensor, my_rank: int,
                      world_size: int, N: int):
    """Halo send/recv CSR + interior mask from one rank's edge list (every dst is one of my atoms).

    Returns (send_offsets [W+1], send_local_indices, recv_offsets [W+1], recv_ghost_indices,
    interior_mask [n_local] bool, recv_atom_global); both CSRs are grouped by peer and ascending in
    global atom id inside a peer."""
    if not edges.is_cuda:
        raise RuntimeError("edges must be a CUDA tensor")
    if edges.dim() != 2 or edges.size(0) != 2:
        raise RuntimeError(f"edges must have shape [2, E], got {list(edges.shape)}")
    if edges.dtype != torch.int64:
        raise RuntimeError("edges must be int64")
    if not pid_outer.is_cuda or pid_outer.dim() != 1:
        raise RuntimeError("pid_outer must be a 1-D CUDA tensor")
    if pid_outer.size(0) != N:
        raise RuntimeError(f"pid_outer must have length N ({N}), got {pid_outer.size(0)}")
    if not my_outer_atoms.is_cuda or my_outer_atoms.dim() != 1 or my_outer_atoms.dtype != torch.int64:
        raise RuntimeError("my_outer_atoms must be 1-D int64 CUDA")
    if world_size < 1:
        raise RuntimeError(f"world_size must be >= 1, got {world_size}")
    if not (0 <= my_rank < world_size):
        raise RuntimeError("my_rank must be in [0, world_size)")
    edges = edges.contiguous()
    pid = pid_outer.to(torch.int64).contiguous()
    mine = my_outer_atoms.contiguous()
    dev = edges.device
    E, W, R = edges.size(1), int(world_size), int(my_rank)
    n_local = mine.numel()
    words = (W + 31) // 32
    L = _lib.lib()
    with torch.cuda.device(dev):
        send_mask = torch.empty((max(N, 1), words), dtype=torch.int32, device=dev)
        recv_mask = torch.empty((max(N, 1), words), dtype=torch.int32, device=dev)
        has_remote = torch.empty((max(N, 1),), dtype=torch.uint8, device=dev)
        bad = torch.zeros((1,), dtype=torch.int32, device=dev)
        _lib.check(L.dynb_halo_mark_from_edges(edges.data_ptr(), E, pid.data_ptr(), N, R, W, send_mask.data_ptr(),
                                               recv_mask.data_ptr(), has_remote.data_ptr(), bad.data_ptr(), _stream(dev)),
                   "halo_mark_from_edges")
        g2l = torch.full((max(N, 1),), -1, dtype=torch.int64, device=dev)
        _lib.check(L.dynb_scatter_iota(mine.data_ptr(), n_local, N, g2l.data_ptr(), bad.data_ptr(), _stream(dev)), "scatter_iota")
        nbytes = ctypes.c_int64()
        _lib.check(L.dynb_csr_workspace_bytes(N, W, ctypes.byref(nbytes)), "csr_workspace_bytes")
        ws_s = scratch(dev, "csr_send", nbytes.value)
        ws_r = scratch(dev, "csr_recv", nbytes.value)
        offs = torch.empty((2, W + 1), dtype=torch.int64, device=dev)
        _lib.check(L.dynb_csr_plan(send_mask.data_ptr(), None, N, R, 2, W, offs[0].data_ptr(), ws_s.data_ptr(), ws_s.numel(),
                                   _stream(dev)), "csr_plan(send)")
        _lib.check(L.dynb_csr_plan(recv_mask.data_ptr(), None, N, R, 2, W, offs[1].data_ptr(), ws_r.data_ptr(), ws_r.numel(),
                                   _stream(dev)), "csr_plan(recv)")
        offs_h = offs.cpu()
        if int(bad.item()) != 0:
            raise RuntimeError("extract_halo_info: an edge endpoint, partition id or my_outer_atoms entry is out of range")
        total_send, total_recv = int(offs_h[0, W]), int(offs_h[1, W])
        send_local = torch.empty((total_send,), dtype=torch.int64, device=dev)
        recv_atom = torch.empty((total_recv,), dtype=torch.int64, device=dev)
        _lib.check(L.dynb_csr_fill(send_mask.data_ptr(), None, N, R, 2, W, g2l.data_ptr(), offs[0].data_ptr(),
                                   send_local.data_ptr(), ws_s.data_ptr(), _stream(dev)), "csr_fill(send)")
        _lib.check(L.dynb_csr_fill(recv_mask.data_ptr(), None, N, R, 2, W, None, offs[1].data_ptr(), recv_atom.data_ptr(),
                                   ws_r.data_ptr(), _stream(dev)), "csr_fill(recv)")
        interior = torch.empty((n_local,), dtype=torch.bool, device=dev)
        _lib.check(L.dynb_gather_not_u8(has_remote.data_ptr(), mine.data_ptr(), n_local, interior.data_ptr(), _stream(dev)),
                   "gather_not_u8")
        recv_ghost = torch.arange(n_local, n_local + total_recv, dtype=torch.int64, device=dev)
        return offs[0].clone(), send_local, offs[1].clone(), recv_ghost, interior, recv_atom
