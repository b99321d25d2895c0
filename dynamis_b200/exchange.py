"""Halo exchange — host side of the reference's ``dynamis_model`` exchange ops.

Names and behaviour follow dynamis_model/src/dynamis_model/comm/exchanger.py:9-536 (``Exchanger``,
``PythonNCCLExchanger``, ``GPUDirectExchanger``), comm/feature_push.py:18-95
(``FeaturePushToExchange``), comm/drift_flags.py, and the compiled ops of
dynamis_model/src/dynamis_model_bindings.cpp:5-105 (``push_buffer_create``, ``FeatureExchanger``).

Two transports behind the same interface:
  * PythonNCCLExchanger — our pack kernel, ``all_to_all_single`` over NCCL straight into the tail
    of the result, our deterministic reverse accumulation kernel.  The per-peer split lists are
    cached per halo plan instead of being read back from the device on every call.
  * GPUDirectExchanger / FeatureExchanger — one-sided push: a single kernel gathers the halo rows
    and stores them into every peer's mapped ghost buffer over NVLink, a release store of the
    generation signals completion and a bounded acquire wait receives it.  Ghost and gradient
    buffers are double-buffered by generation parity, which removes the reference's
    write-after-read hazard on the receiver's buffers.
"""

from __future__ import annotations

import ctypes
import os
from abc import ABC, abstractmethod
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
            # local rows that receive at least one gradient row (for the two-step accumulation)
            self.rows = torch.nonzero(self.inv_offsets[1:] > self.inv_offsets[:-1]).reshape(-1).contiguous()
        self.n_local = n_local

    def add_received(self, recv_ptr: int, out: torch.Tensor) -> None:
        """out (already holding the local gradient rows) += received rows, for the rows that receive any."""
        dev = out.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().dynb_add_rows_listed(self.rows.data_ptr(), self.rows.numel(), out.size(1), _DT[out.dtype], recv_ptr,
                                                       self.inv_offsets.data_ptr(), self.inv_entries.data_ptr(), out.data_ptr(),
                                                       _stream(dev)), "add_rows_listed")

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


# ------------------------------------------------------------------------------------------ one-sided engine
def _align(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


class FeatureExchanger:
    """One-sided halo push over peer-mapped memory.

    Life cycle: ``local_setup`` (allocate and export this rank's buffers) -> exchange the returned
    metadata between ranks -> ``connect`` (map the peers, build the push tables) ->
    ``feature_push_forward`` / ``feature_push_backward`` any number of times -> ``teardown``.
    All ranks must issue the same sequence of pushes.  Forward and backward are each split into
    ``*_begin`` (push + signal) and ``*_end`` (bounded wait + result) so that several ranks can be
    driven from one process on one GPU (all begins, then all ends) without a kernel ever waiting
    for work queued behind it.
    """

    def __init__(self, wait_ns: int = DEFAULT_WAIT_NS):
        self.wait_ns = int(wait_ns)
        self._base = None
        self._setup = False
        self._opened: List[int] = []
        self._gen = [0, 0]  # forward, backward
        self._wired = None

    # -- reference-compatible small surface
    def is_ipc_setup(self) -> bool:
        return self._setup

    def use_fabric(self) -> bool:
        return False

    def set_ce_threshold_bytes(self, t: int) -> None:
        self._ce_threshold = int(t)  # kept for interface parity; this engine always pushes from SMs

    def set_watchdog_flags(self, local_flag: torch.Tensor, global_flag: torch.Tensor) -> None:
        self._wired = (local_flag, global_flag)

    def clear_watchdog_flags(self) -> None:
        self._wired = None

    # -- setup
    def local_setup(self, send_offsets, send_local_indices, recv_offsets, num_local: int, feature_dim: int, rank: int,
                    world_size: int, device: torch.device, dtype: torch.dtype = torch.float32) -> dict:
        if dtype not in _DT:
            raise RuntimeError("FeatureExchanger supports float32 and float64 rows")
        if self._setup or self._base is not None:
            self.teardown()
        self.device = torch.device(device)
        self.rank, self.W = int(rank), int(world_size)
        self.n_local, self.F, self.dtype = int(num_local), int(feature_dim), dtype
        self.row_bytes = self.F * torch.empty((), dtype=dtype).element_size()
        so = [int(v) for v in send_offsets.tolist()]
        ro = [int(v) for v in recv_offsets.tolist()]
        if len(so) != self.W + 1 or len(ro) != self.W + 1:
            raise RuntimeError("send_offsets / recv_offsets must have world_size + 1 entries")
        self.send_offsets_h, self.recv_offsets_h = so, ro
        self.total_send, self.total_recv = so[-1], ro[-1]
        self.send_local = send_local_indices.to(device=self.device, dtype=torch.int64).contiguous()
        if self.send_local.numel() != self.total_send:
            raise RuntimeError("send_local_indices length does not match send_offsets")
        gb = _align(max(self.total_recv, 1) * self.row_bytes)
        rb = _align(max(self.total_send, 1) * self.row_bytes)
        fb = _align(2 * self.W * 4)
        self.ghost_off = [0, gb]
        self.grad_off = [2 * gb, 2 * gb + rb]
        self.flag_off = 2 * gb + 2 * rb
        self.total_bytes = self.flag_off + fb
        L = _lib.lib()
        with torch.cuda.device(self.device):
            p = ctypes.c_void_p()
            _lib.check(L.dynb_ipc_alloc(self.total_bytes, ctypes.byref(p)), "ipc_alloc")
            self._base = p.value
            handle = (ctypes.c_uint8 * 64)()
            _lib.check(L.dynb_ipc_export(self._base, handle), "ipc_export")
            self.reverse = _ReversePlan(self.send_local, self.n_local)
            self.status = torch.zeros((1,), dtype=torch.int32, device=self.device)
            self.status_pin = torch.zeros((1,), dtype=torch.int32).pin_memory()
        return {
            "rank": self.rank, "pid": os.getpid(), "ptr": self._base, "handle": bytes(handle), "device": self.device.index,
            "ghost_off": self.ghost_off, "grad_off": self.grad_off, "flag_off": self.flag_off,
            "send_offsets": so, "recv_offsets": ro, "num_local": self.n_local, "row_bytes": self.row_bytes,
        }

    def connect(self, all_meta: List[dict]) -> None:
        if self._base is None:
            raise RuntimeError("FeatureExchanger: call local_setup() before connect()")
        if len(all_meta) != self.W:
            raise RuntimeError("connect() needs one metadata record per rank")
        L = _lib.lib()
        bases = [0] * self.W
        with torch.cuda.device(self.device):
            for p, m in enumerate(all_meta):
                if m["row_bytes"] != self.row_bytes:
                    raise RuntimeError("ranks disagree on the row size")
                if p == self.rank:
                    bases[p] = self._base
                elif m["pid"] == os.getpid():
                    bases[p] = m["ptr"]  # same process (several ranks driven from one process)
                    if m["device"] != self.device.index:
                        _lib.check(L.dynb_enable_peer_access(int(m["device"])), "enable_peer_access")
                else:
                    q = ctypes.c_void_p()
                    hb = (ctypes.c_uint8 * 64).from_buffer_copy(m["handle"])
                    _lib.check(L.dynb_ipc_open(hb, ctypes.byref(q)), "ipc_open")
                    bases[p] = q.value
                    self._opened.append(q.value)
            # push tables: [direction][parity] -> device array of dynb_push_target
            recs = []
            for parity in (0, 1):
                fwd, bwd = [], []
                for p, m in enumerate(all_meta):
                    if p == self.rank:
                        continue
                    cnt = self.send_offsets_h[p + 1] - self.send_offsets_h[p]
                    if cnt > 0:
                        if m["recv_offsets"][self.rank + 1] - m["recv_offsets"][self.rank] != cnt:
                            raise RuntimeError(f"halo plan mismatch: rank {self.rank} sends {cnt} rows to {p}, which expects "
                                               f"{m['recv_offsets'][self.rank + 1] - m['recv_offsets'][self.rank]}")
                        fwd.append((bases[p] + m["ghost_off"][parity], m["recv_offsets"][self.rank], self.send_offsets_h[p], cnt))
                    cntb = self.recv_offsets_h[p + 1] - self.recv_offsets_h[p]
                    if cntb > 0:
                        bwd.append((bases[p] + m["grad_off"][parity], m["send_offsets"][self.rank], self.recv_offsets_h[p], cntb))
                recs.append((fwd, bwd))
            self.tables = {}
            for parity, (fwd, bwd) in enumerate(recs):
                for name, lst in (("fwd", fwd), ("bwd", bwd)):
                    flat = []
                    for t in lst:
                        flat.extend(t)
                    ten = torch.tensor(flat if flat else [0, 0, 0, 0], dtype=torch.int64).to(self.device)
                    self.tables[(name, parity)] = (ten, len(lst))
            # flag pointers: my slot in every peer's flag array, per direction
            self.flag_ptrs = {}
            for d, name in enumerate(("fwd", "bwd")):
                ptrs = [0 if p == self.rank else bases[p] + all_meta[p]["flag_off"] + (d * self.W + self.rank) * 4
                        for p in range(self.W)]
                self.flag_ptrs[name] = torch.tensor(ptrs, dtype=torch.int64).to(self.device)
            expect = torch.ones((self.W,), dtype=torch.uint8)
            expect[self.rank] = 0
            self.expect = expect.to(self.device)
        self._gen = [0, 0]
        self._setup = True

    def teardown(self) -> None:
        L = _lib.lib()
        if self._base is not None:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                for q in self._opened:
                    L.dynb_ipc_close(q)
                self._opened = []
                L.dynb_ipc_free(self._base)
        self._base = None
        self._setup = False

    def __del__(self):
        try:
            self.teardown()
        except Exception:
            pass

    # -- status
    def check_status(self) -> None:
        """Synchronises and raises if a bounded wait expired since the last check."""
        torch.cuda.synchronize(self.device)
        v = int(self.status.item())
        if v != 0:
            self.status.zero_()
            raise RuntimeError(f"halo exchange timed out on rank {self.rank}: no completion signal from rank {v - 1} "
                               f"within {self.wait_ns / 1e6:.1f} ms")

    # -- one direction
    def _push(self, name: str, x: torch.Tensor, row_index, src_row_base: int, total_rows: int) -> int:
        d = 0 if name == "fwd" else 1
        self._gen[d] += 1
        gen = self._gen[d]
        parity = gen & 1
        L = _lib.lib()
        table, n_t = self.tables[(name, parity)]
        align = 16 if self.row_bytes % 16 == 0 else 4
        st = _stream(self.device)
        _lib.check(L.dynb_push_rows(x.data_ptr(), self.row_bytes, row_index, src_row_base, table.data_ptr(), n_t, total_rows,
                                    align, st), "push_rows")
        _lib.check(L.dynb_signal_peers(self.flag_ptrs[name].data_ptr(), self.W, gen, st), "signal_peers")
        return gen

    def _wait(self, name: str, gen: int) -> None:
        d = 0 if name == "fwd" else 1
        flags = self._base + self.flag_off + d * self.W * 4
        _lib.check(_lib.lib().dynb_wait_flags(flags, self.expect.data_ptr(), self.W, gen, self.wait_ns, self.status.data_ptr(),
                                              _stream(self.device)), "wait_flags")

    def forward_begin(self, local_features: torch.Tensor) -> Tuple[torch.Tensor, int]:
        if not self._setup:
            raise RuntimeError("FeatureExchanger: IPC not set up. Call setup_ipc() first.")
        if local_features.size(0) != self.n_local or local_features.size(1) != self.F:
            raise RuntimeError(f"local_features shape mismatch: expected [{self.n_local}, {self.F}], got "
                               f"[{local_features.size(0)}, {local_features.size(1)}]")
        if local_features.dtype != self.dtype:
            raise RuntimeError(f"local_features dtype mismatch: expected {self.dtype}, got {local_features.dtype}")
        x = local_features.contiguous()
        with torch.cuda.device(self.device):
            out = torch.empty((self.n_local + self.total_recv, self.F), dtype=self.dtype, device=self.device)
            # rows for the peers leave first; the copy of the local rows then runs while they travel
            gen = self._push("fwd", x, self.send_local.data_ptr(), 0, self.total_send)
            _lib.check(_lib.lib().dynb_copy_async(out.data_ptr(), x.data_ptr(), self.n_local * self.row_bytes, _stream(self.device)),
                       "copy_async")
        return out, gen

    def forward_end(self, out: torch.Tensor, gen: int) -> torch.Tensor:
        with torch.cuda.device(self.device):
            self._wait("fwd", gen)
            src = self._base + self.ghost_off[gen & 1]
            _lib.check(_lib.lib().dynb_copy_async(out.data_ptr() + self.n_local * self.row_bytes, src,
                                                  self.total_recv * self.row_bytes, _stream(self.device)), "copy_async")
        return out

    def feature_push_forward(self, local_features: torch.Tensor, partition_info=None) -> torch.Tensor:
        out, gen = self.forward_begin(local_features)
        return self.forward_end(out, gen)

    def backward_begin(self, grad_output: torch.Tensor) -> Tuple[torch.Tensor, int]:
        if not self._setup:
            raise RuntimeError("FeatureExchanger: IPC not set up. Call setup_ipc() first.")
        g = grad_output.contiguous()
        if g.size(0) != self.n_local + self.total_recv or g.size(1) != self.F:
            raise RuntimeError(f"grad_output shape mismatch: expected [{self.n_local + self.total_recv}, {self.F}]")
        with torch.cuda.device(self.device):
            gen = self._push("bwd", g, None, self.n_local, self.total_recv)
            # the local gradient rows are copied while the ghost rows travel; backward_end adds what arrived
            out = torch.empty((self.n_local, self.F), dtype=self.dtype, device=self.device)
            _lib.check(_lib.lib().dynb_copy_async(out.data_ptr(), g.data_ptr(), self.n_local * self.row_bytes, _stream(self.device)),
                       "copy_async")
        return out, gen

    def backward_end(self, out: torch.Tensor, gen: int) -> torch.Tensor:
        with torch.cuda.device(self.device):
            self._wait("bwd", gen)
            self.reverse.add_received(self._base + self.grad_off[gen & 1], out)
        return out

    def feature_push_backward(self, grad_output: torch.Tensor, grad_input_shape=None, partition_info=None) -> torch.Tensor:
        g, gen = self.backward_begin(grad_output)
        return self.backward_end(g, gen)


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

    def __init__(self, group=None, wait_ns: int = DEFAULT_WAIT_NS) -> None:
        super().__init__()
        self.group = group
        self.exchanger = FeatureExchanger(wait_ns)
        self.is_ipc_setup = False
        self.send_buffer = None
        self.grad_recv_buffer = None
        self._wired_flags = None

    def reset_buffers(self):
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
                                          partition_info.recv_offsets, n_local, feature_dim, rank, W, device)
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
