"""Halo exchange — host side of the reference's ``dynamis_model`` exchange ops.

Names and behaviour follow dynamis_model/src/dynamis_model/comm/exchanger.py:9-536 (``Exchanger``,
``PythonNCCLExchanger``, ``GPUDirectExchanger``), comm/feature_push.py:18-95
(``FeaturePushToExchange``), comm/drift_flags.py, and the compiled ops of
dynamis_model/src/dynamis_model_bindings.cpp:5-105 (``push_buffer_create``, ``FeatureExchanger``).

Two transports behind the same interface:
  * PythonNCCLExchanger — our pack kernel, ``all_to_all_single`` over NCCL straight into the tail
    of the result, our deterministic reverse accumulation kernel.  The per-peer split lists are
    cached per halo plan instead of being read back from the device on every call.
  * GPUDirectExchanger / FeatureExchanger — one-sided push in two launches per exchange.  The
    first stores the halo rows into every peer over NVLink while it copies this rank's own rows
    into the head of the result, and ends with the generation signal (which also carries the
    drift-watchdog word); the second is a bounded wait for the peers' signals.  Peers store ghost
    rows straight into the tail of the result tensor: results are handed out from a small ring of
    peer-visible slots, each rank announcing with every signal where its next ghost rows should
    go; when no slot is free (the caller still holds the earlier results) the rows go to a staging
    buffer and are copied once more.  Gradient receive buffers and staging buffers are
    double-buffered by generation parity, which removes the reference's write-after-read hazard
    on the receiver's buffers.
  * IPCExchanger — the reference's low-level object (caller-owned buffers, separate push, signal
    and wait calls) over the same kernels.
"""

from __future__ import annotations

import ctypes
import os
from abc import ABC, abstractmethod
import weakref
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib
from .partition import _stream, scratch

_DT = {torch.float32: _lib.DYNB_F32, torch.float64: _lib.DYNB_F64}
DEFAULT_WAIT_NS = 20_000_000_000


# ------------------------------------------------------------------------------------------ pack
def push_buffer_create(input: torch.Tensor, buffer: torch.Tensor, input_locs: torch.Tensor) -> torch.Tensor:
    """``buffer[i, :] = input[input_locs[i], :]``; returns ``buffer`` (reference: push_buffer.cu:39-105)."""
    for name, t in (("input", input), ("buffer", buffer), ("input_locs", input_locs)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if input.dim() != 2:
        raise RuntimeError("input must have 2 dimensions")
    if buffer.dim() != 2:
        raise RuntimeError("buffer must have 2 dimensions")
    if input_locs.dim() != 1:
        raise RuntimeError("input_locs must have 1 dimension")
    if buffer.size(0) != input_locs.size(0):
        raise RuntimeError("buffer rows must match size of input_locs")
    if buffer.size(1) != input.size(1):
        raise RuntimeError("input and buffer must have same number of columns")
    if input.dtype != torch.float32:
        raise RuntimeError("input datatype must be float32")
    if buffer.dtype != torch.float32:
        raise RuntimeError("buffer datatype must be float32")
    if input_locs.dtype != torch.int64:
        raise RuntimeError("input_locs datatype must be int64")
    _pack(input, input_locs, buffer)
    return buffer


def _pack(x: torch.Tensor, locs: torch.Tensor, out: torch.Tensor) -> None:
    n = locs.numel()
    if n == 0:
        return
    dev = x.device
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().dynb_pack_rows(x.data_ptr(), x.size(0), x.size(1) * x.element_size(), locs.data_ptr(), n,
                                             out.data_ptr(), None, _stream(dev)), "pack_rows")


# ------------------------------------------------------------------------------------------ inverse CSR
class _ReversePlan:
    """For every local row, the positions of the send list that name it (built once per halo plan)."""

    def __init__(self, send_local: torch.Tensor, n_local: int):
        dev = send_local.device
        ts = send_local.numel()
        L = _lib.lib()
        with torch.cuda.device(dev):
            self.inv_offsets = torch.empty((n_local + 1,), dtype=torch.int64, device=dev)
            self.inv_entries = torch.empty((max(ts, 1),), dtype=torch.int32, device=dev)
            bad = torch.zeros((1,), dtype=torch.int32, device=dev)
            nbytes = ctypes.c_int64()
            _lib.check(L.dynb_inverse_csr_workspace_bytes(ts, n_local, ctypes.byref(nbytes)), "inverse_csr_workspace_bytes")
            ws = scratch(dev, "invcsr", nbytes.value)
            _lib.check(L.dynb_inverse_csr(send_local.data_ptr(), ts, n_local, self.inv_offsets.data_ptr(),
                                          self.inv_entries.data_ptr(), bad.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)),
                       "inverse_csr")
            if int(bad.item()) != 0:
                raise RuntimeError("send_local_indices contains an index outside [0, n_local)")
            # local rows that receive at least one gradient row, as a list and as a byte mask
            recv = self.inv_offsets[1:] > self.inv_offsets[:-1]
            self.rows = torch.nonzero(recv).reshape(-1).contiguous()
            self.has_recv = recv.to(torch.uint8).contiguous()
            # first received row of every listed row (read next to the row id instead of behind two more loads)
            self.row_first = self.inv_entries[self.inv_offsets[self.rows]].contiguous() if self.rows.numel() else self.inv_entries[:0]
        self.n_local = n_local

    def apply(self, grad: torch.Tensor, recv_ptr: int, out: torch.Tensor) -> None:
        dev = grad.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().dynb_unpack_add_rows(grad.data_ptr(), self.n_local, grad.size(1), _DT[grad.dtype], recv_ptr,
                                                       self.inv_offsets.data_ptr(), self.inv_entries.data_ptr(), out.data_ptr(),
                                                       _stream(dev)), "unpack_add_rows")


# ------------------------------------------------------------------------------------------ drift flags
@dataclass
class DriftFlags:
    local: torch.Tensor
    global_: torch.Tensor
    n_wired: int = 0


class _DriftRegistry:
    """Process-wide drift-watchdog flag registry (reference: comm/drift_flags.py)."""

    def __init__(self):
        self._reg: Dict[torch.device, DriftFlags] = {}

    @staticmethod
    def _key(device) -> torch.device:
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        return device

    def enable(self, device) -> DriftFlags:
        key = self._key(device)
        self._reg[key] = DriftFlags(local=torch.zeros(1, dtype=torch.int32, device=key),
                                    global_=torch.zeros(1, dtype=torch.int32, device=key))
        return self._reg[key]

    def get(self, device) -> Optional[DriftFlags]:
        return self._reg.get(self._key(device))

    def disable(self, device=None) -> None:
        if device is None:
            self._reg.clear()
        else:
            self._reg.pop(self._key(device), None)


drift_flags = _DriftRegistry()


# ------------------------------------------------------------------------------------------ peer-visible memory
def _align(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


_TYPESTR = {torch.float32: "<f4", torch.float64: "<f8", torch.uint8: "|u1", torch.int32: "<i4"}


class _DeviceView:
    """Lets ``torch.as_tensor`` wrap raw device memory without a copy.  The tensor's storage keeps
    this object alive, so ``owner`` (and a weak reference to the view) tell when nobody uses the
    memory any more."""

    def __init__(self, ptr: int, shape, dtype: torch.dtype, owner=None):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": tuple(int(v) for v in shape), "typestr": _TYPESTR[dtype],
                                         "data": (int(ptr), False), "version": 3, "strides": None}


def _tensor_over(ptr: int, shape, dtype: torch.dtype, device: torch.device, owner=None):
    view = _DeviceView(ptr, shape, dtype, owner)
    return torch.as_tensor(view, device=device), view


class _IpcAllocation:
    """One dynb_ipc_alloc allocation, freed when the last user lets go."""

    def __init__(self, nbytes: int, device: torch.device):
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        p = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_ipc_alloc(self.nbytes, ctypes.byref(p)), "ipc_alloc")
        self.ptr = p.value

    def handle(self) -> bytes:
        h = (ctypes.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_ipc_export(self.ptr, h), "ipc_export")
        return bytes(h)

    def free(self) -> None:
        if self.ptr is not None:
            try:
                with torch.cuda.device(self.device):
                    torch.cuda.synchronize(self.device)
                    _lib.lib().dynb_ipc_free(self.ptr)
            finally:
                self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _open_handle(handle, device: torch.device) -> int:
    hb = (ctypes.c_uint8 * 64).from_buffer_copy(bytes(bytearray(handle)))
    q = ctypes.c_void_p()
    with torch.cuda.device(device):
        _lib.check(_lib.lib().dynb_ipc_open(hb, ctypes.byref(q)), "CUDA ipc_open")
    return q.value


def exchange_layout(n_local: int, total_recv: int, total_send: int, row_bytes: int, world_size: int, ring: int,
                    capacity: Optional[Tuple[int, int, int]] = None) -> dict:
    """Byte offsets inside a rank's exchange allocation; a pure function of the sizes, so that a rank
    can also derive its peers' layouts from their sizes alone.  ``capacity`` = (result rows, ghost rows,
    sent rows) the regions are sized for, when they are to outlive a change of the halo plan."""
    cap_rows, cap_recv, cap_send = capacity if capacity is not None else (n_local + total_recv, total_recv, total_send)
    slot = _align(max(cap_rows, 1) * row_bytes)
    stage = _align(max(cap_recv, 1) * row_bytes)
    grad = _align(max(cap_send, 1) * row_bytes)
    ring_off = 0
    stage_off = ring * slot
    grad_off = stage_off + 2 * stage
    flags_off = grad_off + 2 * grad
    return {"ring": ring, "ring_off": ring_off, "slot_bytes": slot, "ring_tail": ring_off + n_local * row_bytes,
            "stage_off": [stage_off, stage_off + stage], "grad_off": [grad_off, grad_off + grad], "flags_off": flags_off,
            "flags_bytes": _align(3 * 2 * world_size * 16), "total": flags_off + _align(3 * 2 * world_size * 16),
            "capacity": [int(cap_rows), int(cap_recv), int(cap_send)]}


class _HaloContext:
    """Owns the dynb_halo_ctx of one rank: peer table on the device, counters, status words."""

    def __init__(self, device: torch.device, rank: int, world_size: int, local_base: int, local_flags_off: int,
                 peers: List[_lib.HaloPeer], wait_ns: int):
        self.device, self.rank, self.W, self.wait_ns = device, rank, world_size, int(wait_ns)
        L = _lib.lib()
        arr = (_lib.HaloPeer * world_size)(*peers)
        with torch.cuda.device(device):
            self.peers_dev = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(device)
            self.words = torch.zeros((4,), dtype=torch.int32, device=device)  # [0] done counter, [1..2] status
            hp, dp = ctypes.c_void_p(), ctypes.c_void_p()
            _lib.check(L.dynb_host_alloc_mapped(8, ctypes.byref(hp), ctypes.byref(dp)), "host_alloc_mapped")
        self._host_ptr = hp.value
        self.status_host = (ctypes.c_uint32 * 2).from_address(hp.value)
        self.c = _lib.HaloCtx(peers=self.peers_dev.data_ptr(), local_base=local_base, local_flags_off=local_flags_off,
                              done_counter=self.words.data_ptr(), drift_local=None, drift_global=None,
                              status_dev=self.words.data_ptr() + 4, status_host=dp.value, world_size=world_size, rank=rank)
        self._drift = None
        self.failed: Optional[str] = None

    def ref(self):
        return ctypes.byref(self.c)

    def set_drift(self, local_flag: Optional[torch.Tensor], global_flag: Optional[torch.Tensor]) -> None:
        self._drift = (local_flag, global_flag)
        self.c.drift_local = local_flag.data_ptr() if local_flag is not None else None
        self.c.drift_global = global_flag.data_ptr() if global_flag is not None else None

    def poll(self) -> None:
        """No synchronisation: looks at the host copy of the status words, which a kernel whose wait
        ran out (or which met a bad row index) has written by the time the host sees that kernel's
        successors finish."""
        if self.failed is None and self._host_ptr is not None and (self.status_host[0] or self.status_host[1]):
            if self.status_host[0]:
                self.failed = (f"halo exchange timed out on rank {self.rank}: no completion signal from rank "
                               f"{int(self.status_host[0]) - 1} within {self.wait_ns / 1e6:.1f} ms")
            else:
                self.failed = f"halo exchange on rank {self.rank}: a row index of the halo plan is out of range"
        if self.failed is not None:
            raise RuntimeError(self.failed + "; the exchanger must be set up again")

    def check(self) -> None:
        torch.cuda.synchronize(self.device)
        self.poll()

    def close(self) -> None:
        if self._host_ptr is not None:
            _lib.lib().dynb_host_free_mapped(self._host_ptr)
            self._host_ptr = None
            self.status_host = None


def _validate_flag_pair(local_flag: torch.Tensor, global_flag: torch.Tensor) -> None:
    for t in (local_flag, global_flag):
        if not t.is_cuda:
            raise RuntimeError("set_watchdog_flags: flags must be CUDA tensors")
        if t.dtype != torch.int32 or t.numel() != 1 or not t.is_contiguous():
            raise RuntimeError("set_watchdog_flags: flags must be contiguous int32 tensors with one element")


# ------------------------------------------------------------------------------------------ one-sided engine
class FeatureExchanger:
    """One-sided halo push over peer-mapped memory (reference: FeatureExchanger,
    dynamis_model/src/dynamis_model_bindings.cpp:56-105, dynamis_model/src/csrc/exchanger.cu:16-120).

    Two ways to set it up:
      * ``local_setup`` (allocate and export this rank's exchange allocation) -> exchange the returned
        metadata between ranks -> ``connect`` (map the peers, build the push table); or
      * the reference's sequence ``setup_ipc(13 arguments)`` -> ``create_and_export_sync_handle`` ->
        ``setup_sync(all handles)``; the handle that travels is that of the exchange allocation.
    Then ``feature_push_forward`` / ``feature_push_backward`` any number of times, ``teardown``.
    All ranks must issue the same sequence of pushes.  Forward and backward are each split into
    ``*_begin`` (push + local copy + signal, one launch) and ``*_end`` (bounded wait + what depends on
    the peers' rows, one launch) so that several ranks can be driven from one process on one GPU
    (all begins, then all ends) without a kernel ever waiting for work queued behind it.

    ``result_ring``: number of peer-visible result slots.  A forward result is a tensor over one of
    them, so the peers' stores land in the result itself; a slot is reused only after every tensor
    over it has been dropped, and while none is free the exchange falls back to a staging buffer and
    one more copy of the ghost rows (same result).  0 turns the ring off.
    """

    def __init__(self, wait_ns: int = DEFAULT_WAIT_NS, result_ring: int = 3):
        self.wait_ns = int(wait_ns)
        self.ring = int(result_ring)
        self._alloc: Optional[_IpcAllocation] = None
        self._ctx: Optional[_HaloContext] = None
        self._setup = False
        self._opened: List[int] = []
        self._mapped: Dict[bytes, int] = {}   # peers' allocations already mapped, by handle
        self._gen = [0, 0, 0]  # forward, backward, bare handshake
        self._wired = None
        self._ce_threshold = 0
        self._compat = None
        self.layout = None

    # -- reference-compatible small surface
    def is_ipc_setup(self) -> bool:
        return self._setup

    def use_fabric(self) -> bool:
        return False

    @staticmethod
    def supports_fabric_handles(device_id: int = -1) -> bool:
        return False

    def set_ce_threshold_bytes(self, threshold: int) -> None:
        """Rows for a peer travel by copy engine (pack kernel + one peer copy per rank) instead of SM
        stores when some peer's share reaches ``threshold`` bytes; 0 = never (reference:
        ipc_exchanger.cpp:526-569).  Copy-engine pushes go to the staging buffers, so the result ring is
        off while the threshold is set; set it on every rank before the first push."""
        if int(threshold) > 0 and self._gen[0] > 0 and self.ring > 0:
            raise RuntimeError("set_ce_threshold_bytes must be called before the first push")
        self._ce_threshold = int(threshold)

    def ce_threshold_bytes(self) -> int:
        return self._ce_threshold

    def set_watchdog_flags(self, local_flag: torch.Tensor, global_flag: torch.Tensor) -> None:
        """Every signal from now on carries ``local_flag``; after every wait ``global_flag`` holds the
        bitwise OR over all ranks (reference: ipc_exchanger.cpp:784-838)."""
        _validate_flag_pair(local_flag, global_flag)
        self._wired = (local_flag, global_flag)
        if self._ctx is not None:
            self._ctx.set_drift(local_flag, global_flag)

    def clear_watchdog_flags(self) -> None:
        self._wired = None
        if self._ctx is not None:
            self._ctx.set_drift(None, None)

    @staticmethod
    def allocate_ipc_buffer(rows: int, cols: int, device_index: int) -> torch.Tensor:
        return IPCExchanger.allocate_ipc_buffer(rows, cols, device_index)

    def export_ipc_handle(self, buffer: torch.Tensor) -> List[int]:
        return IPCExchanger.export_ipc_handle(self, buffer)

    # -- setup
    def local_setup(self, send_offsets, send_local_indices, recv_offsets, num_local: int, feature_dim: int, rank: int,
                    world_size: int, device: torch.device, dtype: torch.dtype = torch.float32, headroom: float = 0.0) -> dict:
        """Allocates (or keeps) this rank's exchange allocation for the given halo plan and returns the record
        the peers need.  ``headroom`` > 0 sizes the regions for (1 + headroom) x the plan; a later call whose
        plan still fits — same rank, world, row type — keeps the allocation and the peers' mappings of it, so
        that a halo rebuild costs a metadata exchange instead of allocating and mapping gigabytes again.  Every
        rank must call it at the same point of the push sequence; the generation counters start over."""
        if dtype not in _DT:
            raise RuntimeError("FeatureExchanger supports float32 and float64 rows")
        device = torch.device(device)
        so = [int(v) for v in send_offsets.tolist()]
        ro = [int(v) for v in recv_offsets.tolist()]
        W = int(world_size)
        if not 1 <= W <= 128:
            raise RuntimeError("FeatureExchanger supports 1 to 128 ranks")
        if len(so) != W + 1 or len(ro) != W + 1:
            raise RuntimeError("send_offsets / recv_offsets must have world_size + 1 entries")
        row_bytes = int(feature_dim) * torch.empty((), dtype=dtype).element_size()
        n_local, total_send, total_recv = int(num_local), so[-1], ro[-1]
        keep = (self._alloc is not None and self._alloc.ptr is not None and getattr(self, "layout", None) is not None
                and self.device == device and self.rank == int(rank) and self.W == W and self.row_bytes == row_bytes
                and self.dtype == dtype and self.layout["ring"] == self.ring
                and n_local + total_recv <= self.layout["capacity"][0] and total_recv <= self.layout["capacity"][1]
                and total_send <= self.layout["capacity"][2])
        if not keep and (self._setup or self._alloc is not None):
            self.teardown()
        self.device = device
        self.rank, self.W = int(rank), W
        self.n_local, self.F, self.dtype = n_local, int(feature_dim), dtype
        self.row_bytes = row_bytes
        self.send_offsets_h, self.recv_offsets_h = so, ro
        self.total_send, self.total_recv = total_send, total_recv
        self.send_local = send_local_indices.to(device=self.device, dtype=torch.int64).contiguous()
        if self.send_local.numel() != self.total_send:
            raise RuntimeError("send_local_indices length does not match send_offsets")
        if keep:
            cap = tuple(self.layout["capacity"])
            self.layout = exchange_layout(n_local, total_recv, total_send, row_bytes, W, self.ring, cap)
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                # the handshake records start over with the generation counters
                _lib.check(_lib.lib().dynb_fill_zero(self._alloc.ptr + self.layout["flags_off"], self.layout["flags_bytes"],
                                                     _stream(self.device)), "fill_zero")
                torch.cuda.synchronize(self.device)
            self._setup = False
        else:
            cap = None
            if headroom > 0:
                grow = lambda v: int(v * (1.0 + headroom)) + 1024  # noqa: E731
                cap = (grow(n_local + total_recv), grow(total_recv), grow(total_send))
            self.layout = exchange_layout(n_local, total_recv, total_send, row_bytes, W, self.ring, cap)
            self._alloc = _IpcAllocation(self.layout["total"], self.device)
            self._handle = self._alloc.handle()
        with torch.cuda.device(self.device):
            self.reverse = _ReversePlan(self.send_local, self.n_local)
        return {
            "rank": self.rank, "pid": os.getpid(), "ptr": self._alloc.ptr, "handle": self._handle,
            "device": self.device.index, "layout": self.layout, "send_offsets": so, "recv_offsets": ro,
            "num_local": self.n_local, "row_bytes": self.row_bytes,
        }

    def connect(self, all_meta: List[dict]) -> None:
        if self._alloc is None:
            raise RuntimeError("FeatureExchanger: call local_setup() before connect()")
        if len(all_meta) != self.W:
            raise RuntimeError("connect() needs one metadata record per rank")
        L = _lib.lib()
        peers = []
        with torch.cuda.device(self.device):
            for p, m in enumerate(all_meta):
                if m["row_bytes"] != self.row_bytes:
                    raise RuntimeError("ranks disagree on the row size")
                rec = _lib.HaloPeer()
                if p == self.rank:
                    peers.append(rec)
                    continue
                if m.get("pid") == os.getpid() and m.get("ptr") is not None:
                    base = m["ptr"]  # same process (several ranks driven from one process)
                    if m["device"] != self.device.index:
                        _lib.check(L.dynb_enable_peer_access(int(m["device"])), "enable_peer_access")
                else:
                    base = self._mapped.get(m["handle"])
                    if base is None:
                        base = _open_handle(m["handle"], self.device)
                        self._mapped[m["handle"]] = base
                        self._opened.append(base)
                lay = m["layout"]
                cnt = self.send_offsets_h[p + 1] - self.send_offsets_h[p]
                theirs = m["recv_offsets"][self.rank + 1] - m["recv_offsets"][self.rank]
                if theirs != cnt:
                    raise RuntimeError(f"halo plan mismatch: rank {self.rank} sends {cnt} rows to {p}, which expects {theirs}")
                cntb = self.recv_offsets_h[p + 1] - self.recv_offsets_h[p]
                theirs_b = m["send_offsets"][self.rank + 1] - m["send_offsets"][self.rank]
                if theirs_b != cntb:
                    raise RuntimeError(f"halo plan mismatch: rank {self.rank} expects {cntb} rows from {p}, which sends {theirs_b}")
                rec.remote_base = base
                rec.flags_off = lay["flags_off"]
                rec.fwd_ring_tail = lay["ring_tail"]
                rec.fwd_ring_stride = lay["slot_bytes"]
                rec.fwd_stage_off[0], rec.fwd_stage_off[1] = lay["stage_off"]
                rec.fwd_row_offset = m["recv_offsets"][self.rank]
                rec.send_start, rec.send_count = self.send_offsets_h[p], cnt
                rec.bwd_off[0], rec.bwd_off[1] = lay["grad_off"]
                rec.bwd_row_offset = m["send_offsets"][self.rank]
                rec.recv_start, rec.recv_count = self.recv_offsets_h[p], cntb
                peers.append(rec)
            self._peer_recs = peers
            if self._ctx is not None:
                self._ctx.close()
            self._ctx = _HaloContext(self.device, self.rank, self.W, self._alloc.ptr, self.layout["flags_off"], peers, self.wait_ns)
            if self._wired is not None:
                self._ctx.set_drift(*self._wired)
        self._gen = [0, 0, 0]
        self._announced = 0          # where this generation's ghost rows were told to go: 0 staging, s + 1 slot s
        if len(getattr(self, "_slot_refs", [])) != self.ring:
            self._slot_refs = [None] * self.ring     # kept across a re-plan: results still held keep their slots busy
        self._pending: Dict[int, int] = {}
        self._ce_stage = None
        self._setup = True

    # -- the reference's setup sequence
    def setup_ipc(self, x_buffer, grad_recv_buffer, all_x_handles, all_grad_handles, send_offsets, send_local_indices,
                  recv_offsets, all_recv_offsets, all_num_local, num_local, feature_dim, rank, world_size) -> None:
        """Reference signature (dynamis_model/src/csrc/exchanger.cu:16-40).  ``x_buffer`` and
        ``grad_recv_buffer`` (and their handles) are the caller's buffers of the reference protocol; this
        engine keeps its own exchange allocation (result slots, double-buffered receive buffers,
        handshake records), whose handle travels through ``create_and_export_sync_handle`` /
        ``setup_sync``, so those two buffers are only held, never written."""
        for name, t in (("x_buffer", x_buffer), ("grad_recv_buffer", grad_recv_buffer)):
            if not t.is_cuda:
                raise RuntimeError(f"{name} must be a CUDA tensor")
        rank, W = int(rank), int(world_size)
        aro = all_recv_offsets.to("cpu", torch.int64).reshape(W, W + 1).tolist()
        anl = [int(v) for v in all_num_local.to("cpu", torch.int64).reshape(-1).tolist()]
        self._compat = {"aro": aro, "anl": anl, "x": x_buffer, "g": grad_recv_buffer}
        self._meta = self.local_setup(send_offsets.cpu(), send_local_indices, recv_offsets.cpu(), int(num_local), int(feature_dim),
                                      rank, W, x_buffer.device, x_buffer.dtype)

    def create_and_export_sync_handle(self) -> List[int]:
        if self._alloc is None:
            raise RuntimeError("create_and_export_sync_handle: call setup_ipc() first")
        return list(self._alloc.handle())

    def setup_sync(self, all_sync_handles) -> None:
        if self._compat is None or self._alloc is None:
            raise RuntimeError("setup_sync: call setup_ipc() first")
        aro, anl, W = self._compat["aro"], self._compat["anl"], self.W
        metas = []
        for p in range(W):
            if len(all_sync_handles[p]) != 64:
                raise RuntimeError(f"Invalid IPC counter handle size from rank {p}")
            # rank p sends to j what j expects from p
            counts = [aro[j][p + 1] - aro[j][p] for j in range(W)]
            so_p = [0]
            for j in range(W):
                so_p.append(so_p[-1] + (counts[j] if j != p else 0))
            ro_p = aro[p]
            metas.append({"rank": p, "pid": None, "ptr": None, "handle": bytes(bytearray(all_sync_handles[p])),
                          "device": None, "send_offsets": so_p, "recv_offsets": ro_p, "num_local": anl[p],
                          "row_bytes": self.row_bytes,
                          "layout": exchange_layout(anl[p], ro_p[W], so_p[W], self.row_bytes, W, self.ring)})
        metas[self.rank] = self._meta
        self.connect(metas)

    def record_push_complete(self) -> None:
        """A signal without rows (third handshake channel); pairs with ``wait_for_pushes``."""
        self._require()
        self._gen[2] += 1
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_halo_signal(self._ctx.ref(), 2, self._gen[2], 0, _stream(self.device)), "halo_signal")

    def wait_for_pushes(self) -> None:
        self._require()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_halo_wait(self._ctx.ref(), 2, self._gen[2], self.wait_ns, _stream(self.device)), "halo_wait")

    def teardown(self) -> None:
        L = _lib.lib()
        if self._alloc is not None:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                for q in self._opened:
                    L.dynb_ipc_close(q)
                self._opened = []
                self._mapped = {}
            if self._ctx is not None:
                self._ctx.close()
            # tensors handed out over result slots keep the allocation alive; it is freed with the last of them
            self._alloc = None
            self.layout = None
            self._slot_refs = []
        self._ctx = None
        self._compat = None
        self._setup = False

    def __del__(self):
        try:
            self.teardown()
        except Exception:
            pass

    # -- status
    def _require(self) -> None:
        if not self._setup:
            raise RuntimeError("FeatureExchanger: IPC not set up. Call setup_ipc() first.")
        self._ctx.poll()

    def check_status(self) -> None:
        """Synchronises and raises if a bounded wait expired (or a bad row index was met) since set-up."""
        if self._ctx is not None:
            self._ctx.check()

    # -- result slots
    def _slot_free(self, s: int) -> bool:
        r = self._slot_refs[s]
        return r is None or r() is None

    def _pick_next_slot(self, current: int) -> int:
        if self.ring <= 0 or self._ce_threshold > 0:
            return 0
        for s in range(self.ring):
            if s + 1 != current and self._slot_free(s):
                return s + 1
        return 0

    # -- forward
    def forward_begin(self, local_features: torch.Tensor) -> Tuple[torch.Tensor, int]:
        self._require()
        if local_features.size(0) != self.n_local or local_features.size(1) != self.F:
            raise RuntimeError(f"local_features shape mismatch: expected [{self.n_local}, {self.F}], got "
                               f"[{local_features.size(0)}, {local_features.size(1)}]")
        if local_features.dtype != self.dtype:
            raise RuntimeError(f"local_features dtype mismatch: expected {self.dtype}, got {local_features.dtype}")
        x = local_features.contiguous()
        L = _lib.lib()
        self._gen[0] += 1
        gen = self._gen[0]
        mine = self._announced
        nxt = self._pick_next_slot(mine)
        self._announced = nxt
        rows = self.n_local + self.total_recv
        with torch.cuda.device(self.device):
            st = _stream(self.device)
            if mine > 0:
                out, view = _tensor_over(self._alloc.ptr + self.layout["ring_off"] + (mine - 1) * self.layout["slot_bytes"],
                                         (rows, self.F), self.dtype, self.device, owner=self._alloc)
                self._slot_refs[mine - 1] = weakref.ref(view)
            else:
                out = torch.empty((rows, self.F), dtype=self.dtype, device=self.device)
            skip = 0
            if self._ce_threshold > 0 and self.total_send > 0 and any(
                    r.send_count * self.row_bytes >= self._ce_threshold for r in self._peer_recs):
                # copy-engine variant: pack once, one peer copy per rank, then copy + signal only
                if self._ce_stage is None:
                    self._ce_stage = torch.empty((self.total_send, self.F), dtype=self.dtype, device=self.device)
                _lib.check(L.dynb_pack_rows(x.data_ptr(), self.n_local, self.row_bytes, self.send_local.data_ptr(), self.total_send,
                                            self._ce_stage.data_ptr(), self._ctx.c.status_dev + 4, st), "pack_rows")
                for r in self._peer_recs:
                    if r.remote_base and r.send_count > 0:
                        dst = r.remote_base + r.fwd_stage_off[gen & 1] + r.fwd_row_offset * self.row_bytes
                        _lib.check(L.dynb_copy_async(dst, self._ce_stage.data_ptr() + r.send_start * self.row_bytes,
                                                     r.send_count * self.row_bytes, st), "copy_async")
                skip = 1
            _lib.check(L.dynb_halo_forward_begin(self._ctx.ref(), x.data_ptr(), self.n_local, self.row_bytes,
                                                 self.send_local.data_ptr(), self.total_send, out.data_ptr(), gen, nxt, skip, st),
                       "halo_forward_begin")
        self._pending[gen] = mine
        return out, gen

    def forward_end(self, out: torch.Tensor, gen: int) -> torch.Tensor:
        mine = self._pending.pop(gen)
        with torch.cuda.device(self.device):
            if mine == 0 and self.total_recv > 0:
                stage, tail, nbytes = (self._alloc.ptr + self.layout["stage_off"][gen & 1],
                                       out.data_ptr() + self.n_local * self.row_bytes, self.total_recv * self.row_bytes)
            else:
                stage, tail, nbytes = None, None, 0
            _lib.check(_lib.lib().dynb_halo_forward_end(self._ctx.ref(), gen, self.wait_ns, stage, tail, nbytes,
                                                        _stream(self.device)), "halo_forward_end")
        return out

    def feature_push_forward(self, local_features: torch.Tensor, partition_info=None) -> torch.Tensor:
        out, gen = self.forward_begin(local_features)
        return self.forward_end(out, gen)

    # -- reverse
    def backward_begin(self, grad_output: torch.Tensor) -> Tuple[torch.Tensor, int]:
        self._require()
        g = grad_output.contiguous()
        if g.size(0) != self.n_local + self.total_recv or g.size(1) != self.F:
            raise RuntimeError(f"grad_output shape mismatch: expected [{self.n_local + self.total_recv}, {self.F}]")
        if g.dtype != self.dtype:
            raise RuntimeError(f"grad_output dtype mismatch: expected {self.dtype}, got {g.dtype}")
        self._gen[1] += 1
        gen = self._gen[1]
        with torch.cuda.device(self.device):
            out = torch.empty((self.n_local, self.F), dtype=self.dtype, device=self.device)
            _lib.check(_lib.lib().dynb_halo_backward_begin(self._ctx.ref(), g.data_ptr(), self.n_local, self.total_recv,
                                                           self.row_bytes, self.reverse.has_recv.data_ptr(), out.data_ptr(), gen,
                                                           _stream(self.device)), "halo_backward_begin")
        self._pending[-gen] = g  # the second half reads the gradient rows again
        return out, gen

    def backward_end(self, out: torch.Tensor, gen: int) -> torch.Tensor:
        g = self._pending.pop(-gen)
        rv = self.reverse
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_halo_backward_end(self._ctx.ref(), gen, self.wait_ns, g.data_ptr(), rv.rows.data_ptr(),
                                                         rv.row_first.data_ptr(), rv.rows.numel(), self.F, _DT[self.dtype],
                                                         self._alloc.ptr + self.layout["grad_off"][gen & 1],
                                                         rv.inv_offsets.data_ptr(), rv.inv_entries.data_ptr(), out.data_ptr(),
                                                         _stream(self.device)), "halo_backward_end")
        return out

    def feature_push_backward(self, grad_output: torch.Tensor, grad_input_shape=None, partition_info=None) -> torch.Tensor:
        g, gen = self.backward_begin(grad_output)
        return self.backward_end(g, gen)


class IPCExchanger:
    """The reference's low-level exchange object (dynamis_model/src/dynamis_model_bindings.cpp:13-54,
    dynamis_model/src/csrc/exchange/ipc_exchanger.cpp:117-952) with its call sequence: the caller owns
    ``x_buffer`` [n_local + n_ghost, F] and ``grad_recv_buffer`` [total_send, F] (from
    ``allocate_ipc_buffer``), pushes, signals and waits in separate calls.  Differences: the signal
    stores a record into every peer instead of bumping a local counter that peers poll remotely, the
    wait is bounded (``wait_ns``; on expiry the next call raises), and bad row indices are reported
    instead of written."""

    MAX_RANKS = 128

    def __init__(self, wait_ns: int = DEFAULT_WAIT_NS):
        self.wait_ns = int(wait_ns)
        self._is_setup = False
        self._sync: Optional[_IpcAllocation] = None
        self._ctx: Optional[_HaloContext] = None
        self._opened: List[int] = []
        self._gen = 0
        self._wired = None

    @staticmethod
    def supports_fabric_handles(device_id: int = -1) -> bool:
        return False

    @staticmethod
    def allocate_ipc_buffer(rows: int, cols: int, device_index: int) -> torch.Tensor:
        if rows < 0 or cols < 0:
            raise RuntimeError("rows and cols must be non-negative")
        dev = torch.device("cuda", int(device_index))
        alloc = _IpcAllocation(max(rows * cols * 4, 4), dev)
        t, _ = _tensor_over(alloc.ptr, (rows, cols), torch.float32, dev, owner=alloc)
        return t

    def export_ipc_handle(self, buffer: torch.Tensor) -> List[int]:
        if not buffer.is_cuda:
            raise RuntimeError("export_ipc_handle: buffer must be a CUDA tensor")
        h = (ctypes.c_uint8 * 64)()
        with torch.cuda.device(buffer.device):
            _lib.check(_lib.lib().dynb_ipc_export(buffer.data_ptr(), h), "CUDA ipc_export")
        return list(bytes(h))

    def setup(self, x_buffer, grad_recv_buffer, all_x_handles, all_grad_handles, send_offsets, send_local_indices, recv_offsets,
              all_recv_offsets, all_num_local, num_local, feature_dim, rank, world_size) -> None:
        if self._is_setup:
            self.teardown()
        dev = x_buffer.device
        self.device, self.rank, self.W = dev, int(rank), int(world_size)
        if not 1 <= self.W <= self.MAX_RANKS:
            raise RuntimeError("IPCExchanger supports 1 to 128 ranks")
        self.F, self.n_local = int(feature_dim), int(num_local)
        self.row_bytes = self.F * 4
        so = [int(v) for v in send_offsets.cpu().tolist()]
        ro = [int(v) for v in recv_offsets.cpu().tolist()]
        aro = all_recv_offsets.to("cpu", torch.int64).reshape(self.W, self.W + 1).tolist()
        anl = [int(v) for v in all_num_local.to("cpu", torch.int64).reshape(-1).tolist()]
        self.total_send, self.total_recv = so[self.W], ro[self.W]
        self.send_local = send_local_indices.to(device=dev, dtype=torch.int64).contiguous()
        self._x, self._g = x_buffer, grad_recv_buffer
        fwd, bwd = [], []
        for r in range(self.W):
            if r == self.rank:
                continue
            if len(all_x_handles[r]) != 64:
                raise RuntimeError(f"Invalid IPC handle size from rank {r}")
            if len(all_grad_handles[r]) != 64:
                raise RuntimeError(f"Invalid IPC grad handle size from rank {r}")
            xp, gp = _open_handle(all_x_handles[r], dev), _open_handle(all_grad_handles[r], dev)
            self._opened += [xp, gp]
            # forward: my rows for r land behind r's own rows, at r's receive offset for me
            fwd += [xp, anl[r] + aro[r][self.rank], so[r], so[r + 1] - so[r], anl[r] + aro[r][self.W]]
            # reverse: the gradient rows of r's atoms land in r's receive buffer at r's send offset for me
            off = sum(aro[j][r + 1] - aro[j][r] for j in range(self.rank))
            tot = sum(aro[j][r + 1] - aro[j][r] for j in range(self.W))
            bwd += [gp, off, ro[r], ro[r + 1] - ro[r], tot]
        with torch.cuda.device(dev):
            self._fwd = torch.tensor(fwd if fwd else [0] * 5, dtype=torch.int64).to(dev)
            self._bwd = torch.tensor(bwd if bwd else [0] * 5, dtype=torch.int64).to(dev)
            self._bad = torch.zeros((1,), dtype=torch.int32, device=dev)
        self._n_targets = self.W - 1
        self._is_setup = True

    def _push(self, x: torch.Tensor, table: torch.Tensor, index, base: int, total: int) -> None:
        if not (x.is_cuda and x.is_contiguous()):
            raise RuntimeError("x_buffer must be contiguous CUDA tensor")
        if self._ctx is not None:
            self._ctx.poll()
        if total == 0 or self._n_targets == 0:
            return
        align = 16 if self.row_bytes % 16 == 0 else 4
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_push_rows(x.data_ptr(), x.size(0), self.row_bytes, index, base, table.data_ptr(),
                                                 self._n_targets, total, align, self._bad.data_ptr(), _stream(self.device)),
                       "push_rows")

    def push_forward(self, x_buffer: torch.Tensor) -> None:
        if not self._is_setup:
            raise RuntimeError("IPCExchanger::push_forward: not set up")
        self._push(x_buffer, self._fwd, self.send_local.data_ptr(), 0, self.total_send)

    def push_backward(self, grad_at_ghost: torch.Tensor) -> None:
        if not self._is_setup:
            raise RuntimeError("IPCExchanger::push_backward: not set up")
        self._push(grad_at_ghost, self._bwd, None, self.n_local, self.total_recv)

    def create_and_export_sync_handle(self) -> List[int]:
        dev = self.device if self._is_setup else torch.device("cuda", torch.cuda.current_device())
        if self._ctx is not None:
            self._ctx.close()
            self._ctx = None
        self._sync = _IpcAllocation(_align(3 * 2 * self.MAX_RANKS * 16), dev)
        self._gen = 0
        return list(self._sync.handle())

    def setup_sync(self, all_sync_handles) -> None:
        if self._sync is None or not self._is_setup:
            raise RuntimeError("setup_sync: call setup() and create_and_export_sync_handle() first")
        peers = []
        for r in range(self.W):
            rec = _lib.HaloPeer()
            if r != self.rank:
                if len(all_sync_handles[r]) != 64:
                    raise RuntimeError(f"Invalid IPC counter handle size from rank {r}")
                base = _open_handle(all_sync_handles[r], self.device)
                self._opened.append(base)
                rec.remote_base, rec.flags_off = base, 0
            peers.append(rec)
        self._ctx = _HaloContext(self.device, self.rank, self.W, self._sync.ptr, 0, peers, self.wait_ns)
        if self._wired is not None:
            self._ctx.set_drift(*self._wired)

    def record_push_complete(self) -> None:
        if self._ctx is None:
            raise RuntimeError("record_push_complete: counter not set up")
        self._ctx.poll()
        self._gen += 1
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_halo_signal(self._ctx.ref(), 2, self._gen, 0, _stream(self.device)), "halo_signal")

    def wait_for_pushes(self) -> None:
        if self._ctx is None:
            raise RuntimeError("wait_for_pushes: counter not set up")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_halo_wait(self._ctx.ref(), 2, self._gen, self.wait_ns, _stream(self.device)), "halo_wait")

    def set_watchdog_flags(self, local_flag: torch.Tensor, global_flag: torch.Tensor) -> None:
        _validate_flag_pair(local_flag, global_flag)
        self._wired = (local_flag, global_flag)
        if self._ctx is not None:
            self._ctx.set_drift(local_flag, global_flag)

    def clear_watchdog_flags(self) -> None:
        self._wired = None
        if self._ctx is not None:
            self._ctx.set_drift(None, None)

    def check_status(self) -> None:
        if self._ctx is not None:
            self._ctx.check()
        if self._is_setup and int(self._bad.item()) != 0:
            raise RuntimeError("IPCExchanger: a row index of the halo plan is out of range")

    def teardown(self) -> None:
        if self._is_setup or self._sync is not None:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                for q in self._opened:
                    _lib.lib().dynb_ipc_close(q)
            self._opened = []
        if self._ctx is not None:
            self._ctx.close()
            self._ctx = None
        self._sync = None
        self._is_setup = False

    def is_setup(self) -> bool:
        return self._is_setup

    def use_fabric(self) -> bool:
        return False

    def __del__(self):
        try:
            self.teardown()
        except Exception:
            pass


def supports_fabric_handles(device_id: int = -1) -> bool:
    """Multi-node fabric handles are not used by this implementation (one NVSwitch domain, CUDA IPC)."""
    return False


# ------------------------------------------------------------------------------------------ Exchanger classes
class Exchanger(ABC):
    def __init__(self) -> None:
        super().__init__()
        self.is_ipc_setup = False

    @abstractmethod
    def setup_exchanger(self, feature_dim: int, partition_info, device: torch.device): ...

    @abstractmethod
    def reset_buffers(self): ...

    @abstractmethod
    def feature_push_impl(self, features_to_push: torch.Tensor, partition_info) -> torch.Tensor: ...

    @abstractmethod
    def feature_push_backward_impl(self, grad_output: torch.Tensor, input_feature_shape, partition_info) -> torch.Tensor: ...

    @staticmethod
    def _is_single_rank() -> bool:
        import torch.distributed as dist

        return dist.is_initialized() and dist.get_world_size() == 1

    def feature_push_forward(self, features_to_push: torch.Tensor, partition_info) -> torch.Tensor:
        if self._is_single_rank():
            return features_to_push
        if not self.is_ipc_setup:
            self.setup_exchanger(features_to_push.shape[-1], partition_info, features_to_push.device)
            self.is_ipc_setup = True
        return self.feature_push_impl(features_to_push, partition_info)

    def feature_push_backward(self, grad_output: torch.Tensor, input_feature_shape, partition_info) -> torch.Tensor:
        if self._is_single_rank():
            return grad_output
        if not self.is_ipc_setup:
            raise RuntimeError("Exchanger is not setup for backward pass. Call feature_push_forward first.")
        return self.feature_push_backward_impl(grad_output, input_feature_shape, partition_info)


class _PlanCache:
    """Host copies of a halo plan's split lists and its reverse plan, keyed by the plan's tensors."""

    def __init__(self):
        self.key = None

    def get(self, info, n_local: int, device):
        key = (info.send_offsets.data_ptr(), info.send_offsets._version, info.recv_offsets.data_ptr(),
               info.recv_offsets._version, info.send_local_indices.data_ptr(), n_local)
        if key != self.key:
            so = info.send_offsets.cpu().tolist()
            ro = info.recv_offsets.cpu().tolist()
            W = len(so) - 1
            self.send_splits = [so[r + 1] - so[r] for r in range(W)]
            self.recv_splits = [ro[r + 1] - ro[r] for r in range(W)]
            self.total_send, self.total_recv = so[-1], ro[-1]
            self.send_local = info.send_local_indices.to(device=device, dtype=torch.int64).contiguous()
            self.reverse = _ReversePlan(self.send_local, n_local) if self.send_local.numel() else None
            self.key = key
        return self


class PythonNCCLExchanger(Exchanger):
    """Pack kernel -> NCCL all_to_all_single into the tail of the result -> reverse accumulation kernel."""

    def __init__(self, group=None) -> None:
        super().__init__()
        self.group = group
        self.send_buffer: Optional[torch.Tensor] = None
        self.grad_recv_buffer: Optional[torch.Tensor] = None
        self._cache = _PlanCache()

    def setup_exchanger(self, feature_dim, partition_info, device) -> None:
        import torch.distributed as dist

        assert dist.is_initialized(), "Distributed process group is not initialized"
        self.is_ipc_setup = True

    def reset_buffers(self):
        self.send_buffer = None
        self.grad_recv_buffer = None
        self._cache = _PlanCache()
        self.is_ipc_setup = False

    def feature_push_impl(self, features_to_push, partition_info):
        import torch.distributed as dist

        x = features_to_push.contiguous()
        dev, n_local, F = x.device, x.shape[0], x.shape[1]
        c = self._cache.get(partition_info, n_local, dev)
        out = torch.empty((n_local + c.total_recv, F), dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().dynb_copy_async(out.data_ptr(), x.data_ptr(), n_local * F * x.element_size(), _stream(dev)),
                       "copy_async")
        if self.send_buffer is None or self.send_buffer.shape != (c.total_send, F) or self.send_buffer.dtype != x.dtype:
            self.send_buffer = torch.empty((c.total_send, F), dtype=x.dtype, device=dev)
        _pack(x, c.send_local, self.send_buffer)
        dist.all_to_all_single(out[n_local:], self.send_buffer, c.recv_splits, c.send_splits, group=self.group)
        return out

    def feature_push_backward_impl(self, grad_output, input_feature_shape, partition_info):
        import torch.distributed as dist

        g = grad_output.contiguous()
        dev = g.device
        n_local, F = int(input_feature_shape[0]), int(input_feature_shape[1])
        c = self._cache.get(partition_info, n_local, dev)
        if self.grad_recv_buffer is None or self.grad_recv_buffer.shape != (c.total_send, F) or self.grad_recv_buffer.dtype != g.dtype:
            self.grad_recv_buffer = torch.empty((c.total_send, F), dtype=g.dtype, device=dev)
        dist.all_to_all_single(self.grad_recv_buffer, g[n_local:n_local + c.total_recv], c.send_splits, c.recv_splits,
                               group=self.group)
        out = torch.empty((n_local, F), dtype=g.dtype, device=dev)
        if c.reverse is not None and g.dtype in _DT:
            c.reverse.apply(g, self.grad_recv_buffer.data_ptr(), out)
        elif c.reverse is None:
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().dynb_copy_async(out.data_ptr(), g.data_ptr(), n_local * F * g.element_size(), _stream(dev)),
                           "copy_async")
        else:
            raise RuntimeError("reverse halo accumulation supports float32 and float64")
        return out


class GPUDirectExchanger(Exchanger):
    """One-sided NVLink push (wraps FeatureExchanger; metadata travels through torch.distributed)."""

    def __init__(self, group=None, wait_ns: int = DEFAULT_WAIT_NS, result_ring: int = 3, headroom: float = 0.0) -> None:
        super().__init__()
        self.group = group
        self.headroom = float(headroom)   # > 0: set_up again for a new halo plan keeps allocation and mappings while it fits
        self.exchanger = FeatureExchanger(wait_ns, result_ring)
        self.is_ipc_setup = False
        self.send_buffer = None
        self.grad_recv_buffer = None
        self._wired_flags = None

    def reset_buffers(self):
        try:
            self.exchanger.check_status()  # a wait that ran out since the last push is reported here at the latest
        finally:
            self.exchanger.teardown()
            self.send_buffer = None
            self.grad_recv_buffer = None
            self.is_ipc_setup = False

    def _wire_drift_flags(self, device) -> None:
        flags = drift_flags.get(device)
        if flags is self._wired_flags:
            return
        if flags is None:
            self.exchanger.clear_watchdog_flags()
        else:
            self.exchanger.set_watchdog_flags(flags.local, flags.global_)
            flags.n_wired += 1
        self._wired_flags = flags

    def setup_exchanger(self, feature_dim, partition_info, device):
        import torch.distributed as dist

        assert dist.is_initialized(), "Distributed process group is not initialized"
        if self._is_single_rank():
            self.is_ipc_setup = True
            return
        rank, W = dist.get_rank(self.group), dist.get_world_size(self.group)
        n_local = len(partition_info.partition_indices)
        meta = self.exchanger.local_setup(partition_info.send_offsets, partition_info.send_local_indices,
                                          partition_info.recv_offsets, n_local, feature_dim, rank, W, device,
                                          headroom=self.headroom)
        all_meta = [None] * W
        dist.all_gather_object(all_meta, meta, group=self.group)
        self.exchanger.connect(all_meta)
        dist.barrier(group=self.group)
        self.is_ipc_setup = True

    def feature_push_impl(self, features_to_push, partition_info):
        self._wire_drift_flags(features_to_push.device)
        return self.exchanger.feature_push_forward(features_to_push, partition_info)

    def feature_push_backward_impl(self, grad_output, input_feature_shape, partition_info):
        self._wire_drift_flags(grad_output.device)
        return self.exchanger.feature_push_backward(grad_output, input_feature_shape, partition_info)


class FeaturePushToExchange(torch.autograd.Function):
    """Autograd bridge: forward returns [local | ghost] rows, backward returns the ghost rows'
    gradients to their owners and adds them in (reference: comm/feature_push.py:18-95)."""

    @staticmethod
    def forward(ctx, features_to_push: torch.Tensor, state, exchanger: Exchanger) -> torch.Tensor:
        ctx._state = state
        ctx._features_to_push_shape = features_to_push.shape
        ctx._exchanger = exchanger
        assert features_to_push.dim() == 2, (
            "features_to_push must be 2-D [n_local, feature_dim], got shape " f"{tuple(features_to_push.shape)}")
        return exchanger.feature_push_forward(features_to_push, state.local_partition_info)

    @staticmethod
    def backward(ctx, grad_output):
        g = ctx._exchanger.feature_push_backward(grad_output, ctx._features_to_push_shape, ctx._state.local_partition_info)
        return g, None, None
