"""ctypes binding of libdynb.so (the C ABI declared in include/dynb.h).

The library is the product: there is no fallback.  If it has not been built, importing
``lib()`` raises with the build command.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libdynb.so")

DYNB_F32 = 0
DYNB_F64 = 1

RG_SRC_OVERFLOW = 1
RG_BAD_TARGET = 2
RG_SHIFT_RANGE = 4
RG_NONFINITE = 8

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int
_f64 = ctypes.c_double
_u32 = ctypes.c_uint32


class RgHeader(ctypes.Structure):
    _fields_ = [
        ("E", ctypes.c_int64),
        ("M", ctypes.c_int64),
        ("status", ctypes.c_uint32),
        ("max_degree", ctypes.c_uint32),
        ("grid", ctypes.c_int32 * 3),
        ("group_cells", ctypes.c_int32),
        ("num_groups", ctypes.c_int64),
        ("reserved", ctypes.c_int64 * 2),
    ]


class HaloPeer(ctypes.Structure):
    """dynb_halo_peer"""
    _fields_ = [
        ("remote_base", ctypes.c_void_p),
        ("flags_off", ctypes.c_int64),
        ("fwd_ring_tail", ctypes.c_int64),
        ("fwd_ring_stride", ctypes.c_int64),
        ("fwd_stage_off", ctypes.c_int64 * 2),
        ("fwd_row_offset", ctypes.c_int64),
        ("send_start", ctypes.c_int64),
        ("send_count", ctypes.c_int64),
        ("bwd_off", ctypes.c_int64 * 2),
        ("bwd_row_offset", ctypes.c_int64),
        ("recv_start", ctypes.c_int64),
        ("recv_count", ctypes.c_int64),
    ]


class HaloCtx(ctypes.Structure):
    """dynb_halo_ctx"""
    _fields_ = [
        ("peers", ctypes.c_void_p),
        ("local_base", ctypes.c_void_p),
        ("local_flags_off", ctypes.c_int64),
        ("done_counter", ctypes.c_void_p),
        ("drift_local", ctypes.c_void_p),
        ("drift_global", ctypes.c_void_p),
        ("status_dev", ctypes.c_void_p),
        ("status_host", ctypes.c_void_p),
        ("world_size", ctypes.c_int32),
        ("rank", ctypes.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/dynb.h declares must be listed here
SIGNATURES = {
    "dynb_last_error": (ctypes.c_char_p, []),
    "dynb_version": (_i32, []),
    "dynb_rg_suggest_capacity": (_i32, [_i64, _p, _p, _f64, _i32, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "dynb_rg_workspace_bytes": (_i32, [_i64, _i64, _i64, _i64, _i32, ctypes.POINTER(_i64)]),
    "dynb_rg_plan": (_i32, [_p, _i32, _i64, _p, _p, _f64, _p, _i64, _p, _i64, _i64, _i64, _p, _p, _p]),
    "dynb_rg_fill": (_i32, [_p, _i32, _p, _p, _p, _i64, _p]),
    "dynb_rg_fill_glue": (_i32, [_p, _i32, _p, _p, _p, _p, _i32, _p, _i64, _p]),
    "dynb_rg_halo_mark": (_i32, [_p, _i32, _p, _i64, _i64, _p, _p, _p]),
    "dynb_sfc_workspace_bytes": (_i32, [_i64, ctypes.POINTER(_i64)]),
    "dynb_sfc_partition": (_i32, [_p, _i64, _p, _i64, _i32, _p, _p, _p, _i64, _p]),
    "dynb_sfc_keys": (_i32, [_p, _i64, _i32, _p, _p, _i64, _p]),
    "dynb_sfc_minmax": (_i32, [_p, _i64, _p, _p]),
    "dynb_sfc_keys_from_bounds": (_i32, [_p, _i64, _i32, _p, _p, _p]),
    "dynb_label_by_splits": (_i32, [_p, _p, _i64, _p, _p, _i32, _p, _p]),
    "dynb_radix_sort_workspace_bytes": (_i32, [_i64, ctypes.POINTER(_i64)]),
    "dynb_radix_sort_pairs": (_i32, [_p, _p, _i64, _i32, _i32, _p, _i64, _p]),
    "dynb_bincount_i64": (_i32, [_p, _i64, _i64, _p, _p, _p]),
    "dynb_select_workspace_bytes": (_i32, [_i64, ctypes.POINTER(_i64)]),
    "dynb_select_eq_i64": (_i32, [_p, _i64, _i64, _p, _p, _p, _p, _i64, _p]),
    "dynb_halo_mark_from_edges": (_i32, [_p, _i64, _p, _i64, _i64, _i64, _p, _p, _p, _p, _p]),
    "dynb_csr_workspace_bytes": (_i32, [_i64, _i64, ctypes.POINTER(_i64)]),
    "dynb_csr_plan": (_i32, [_p, _p, _i64, _i64, _i32, _i64, _p, _p, _i64, _p]),
    "dynb_csr_fill": (_i32, [_p, _p, _i64, _i64, _i32, _i64, _p, _p, _p, _p, _p]),
    "dynb_gather_not_u8": (_i32, [_p, _p, _i64, _p, _p]),
    "dynb_scatter_iota": (_i32, [_p, _i64, _i64, _p, _p, _p]),
    "dynb_filter_edges_plan": (_i32, [_p, _p, _p, _p, _f64, _i64, _p, _p, _i64, _p]),
    "dynb_filter_edges_fill": (_i32, [_p, _p, _i32, _i64, _i64, _p, _p, _p, _p]),
    "dynb_pack_rows": (_i32, [_p, _i64, _i64, _p, _i64, _p, _p, _p]),
    "dynb_push_rows": (_i32, [_p, _i64, _i64, _p, _i64, _p, _i32, _i64, _i32, _p, _p]),
    "dynb_halo_forward_begin": (_i32, [_p, _p, _i64, _i64, _p, _i64, _p, _u32, _u32, _i32, _p]),
    "dynb_halo_forward_end": (_i32, [_p, _u32, _i64, _p, _p, _i64, _p]),
    "dynb_halo_backward_begin": (_i32, [_p, _p, _i64, _i64, _i64, _p, _p, _u32, _p]),
    "dynb_halo_backward_end": (_i32, [_p, _u32, _i64, _p, _p, _p, _i64, _i64, _i32, _p, _p, _p, _p, _p]),
    "dynb_halo_signal": (_i32, [_p, _i32, _u32, _u32, _p]),
    "dynb_halo_wait": (_i32, [_p, _i32, _u32, _i64, _p]),
    "dynb_host_alloc_mapped": (_i32, [_i64, ctypes.POINTER(_p), ctypes.POINTER(_p)]),
    "dynb_host_free_mapped": (_i32, [_p]),
    "dynb_inverse_csr_workspace_bytes": (_i32, [_i64, _i64, ctypes.POINTER(_i64)]),
    "dynb_inverse_csr": (_i32, [_p, _i64, _i64, _p, _p, _p, _p, _i64, _p]),
    "dynb_unpack_add_rows": (_i32, [_p, _i64, _i64, _i32, _p, _p, _p, _p, _p]),
    "dynb_ipc_alloc": (_i32, [_i64, ctypes.POINTER(_p)]),
    "dynb_ipc_free": (_i32, [_p]),
    "dynb_ipc_export": (_i32, [_p, _p]),
    "dynb_ipc_open": (_i32, [_p, ctypes.POINTER(_p)]),
    "dynb_ipc_close": (_i32, [_p]),
    "dynb_enable_peer_access": (_i32, [_i32]),
    "dynb_copy_async": (_i32, [_p, _p, _i64, _p]),
    "dynb_fill_zero": (_i32, [_p, _i64, _p]),
    "dynb_scatter_rows": (_i32, [_p, _i64, _p, _i64, _i64, _p, _p, _p]),
    "dynb_drift_flag": (_i32, [_p, _p, _p, _p, _i64, _f64, _f64, _p, _p, _p]),
    "dynb_kdtree_workspace_bytes": (_i32, [_i64, _i64, ctypes.POINTER(_i64)]),
    "dynb_kdtree_partition": (_i32, [_p, _i64, _p, _i64, _p, _i32, _p, _i64, _p]),
    "dynb_integrator_step": (_i32, [_i32, _p, _p, _p, _p, _p, _i64, _f64, _f64, _f64, _p, _p, _f64, _p, _p, _p]),
    "dynb_sfc_static_max_atoms": (_i64, []),
    "dynb_sfc_partition_static": (_i32, [_p, _i64, _p, _i64, _i32, _p, _p, _p]),
}

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(
                f"{SO_PATH} is missing: build the CUDA library first with `python -m dynamis_b200.build` "
                "(there is no CPU or PyTorch fallback)"
            )
        L = ctypes.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().dynb_last_error()
        text = msg.decode() if msg else ""
        raise RuntimeError(f"dynb {what} failed (code {rc}): {text}")


class _NoSwitch:
    """Context manager that does nothing (the device is already the current one)."""

    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def on_device(dev):
    """``torch.cuda.device(dev)``, or a no-op context when ``dev`` is the current device already: entering and
    leaving the real guard costs several microseconds of host time in front of every launch sequence."""
    import torch

    index = dev.index if dev.index is not None else torch.cuda.current_device()
    if torch.cuda.current_device() == index:
        return _NO_SWITCH
    return torch.cuda.device(index)
