"""GPU test of dynb_sfc_partition_static, the entry point for callers that cannot allocate device
memory while they run (their host owns the allocator, or a cudaMalloc's device-wide synchronisation
is not acceptable in their loop).  It keeps its scratch in a fixed array inside the library.

Called through the C ABI and compared, label for label, with dynb_sfc_partition (which takes a
caller-provided workspace) on two calls in a row — the second one smaller and weighted, so that stale
scratch contents from the first call would show.  Collected last on purpose (file name), and it must
pass both alone in a fresh process and after every other test."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(L, pos, weights, W, curve, dev):
    from dynamis_b200 import _lib

    n = pos.size(0)
    st = torch.cuda.current_stream(dev).cuda_stream
    wp = weights.data_ptr() if weights is not None else None
    a = torch.full((n,), -1, dtype=torch.int64, device=dev)
    pa = torch.full((n,), -1, dtype=torch.int64, device=dev)
    _lib.check(L.dynb_sfc_partition_static(pos.data_ptr(), n, wp, W, curve, a.data_ptr(), pa.data_ptr(), st), "sfc_partition_static")
    nbytes = ctypes.c_int64()
    _lib.check(L.dynb_sfc_workspace_bytes(n, ctypes.byref(nbytes)), "sfc_workspace_bytes")
    ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
    b = torch.full((n,), -2, dtype=torch.int64, device=dev)
    pb = torch.full((n,), -2, dtype=torch.int64, device=dev)
    _lib.check(L.dynb_sfc_partition(pos.data_ptr(), n, wp, W, curve, b.data_ptr(), pb.data_ptr(), ws.data_ptr(), ws.numel(), st),
               "sfc_partition")
    torch.cuda.synchronize(dev)
    return a, pa, b, pb


def test_static_scratch_partition_matches_workspace_partition(cuda):
    from dynamis_b200 import _lib

    L = _lib.lib()
    max_atoms = int(L.dynb_sfc_static_max_atoms())
    assert max_atoms == 131072
    g = torch.Generator(device="cpu").manual_seed(11)
    with torch.cuda.device(cuda):
        # call 1: the largest size the built-in scratch takes, Morton, unweighted
        pos1 = (torch.rand(max_atoms, 3, generator=g) * 90.0).to(cuda)
        a, pa, b, pb = _both(L, pos1, None, 8, 0, cuda)
        assert torch.equal(a, b) and torch.equal(pa, pb)
        assert a.min() >= 0 and a.max() == 7
        # call 2, directly after: smaller, weighted, the other curve — reuses the same scratch
        pos2 = (torch.rand(30_001, 3, generator=g) * 40.0).to(cuda)
        w2 = torch.randint(1, 500, (30_001,), generator=g).to(cuda)
        a, pa, b, pb = _both(L, pos2, w2, 5, 1, cuda)
        assert torch.equal(a, b) and torch.equal(pa, pb)
        a, pa, b, pb = _both(L, pos2, w2, 5, 0, cuda)
        assert torch.equal(a, b) and torch.equal(pa, pb)
        # without the permutation output (dynb_sfc_partition then selects the split points without a sort when
        # it has its full workspace; the built-in scratch always sorts): same labels
        st = torch.cuda.current_stream(cuda).cuda_stream
        c = torch.full((30_001,), -3, dtype=torch.int64, device=cuda)
        _lib.check(L.dynb_sfc_partition_static(pos2.data_ptr(), 30_001, w2.data_ptr(), 5, 0, c.data_ptr(), None, st),
                   "sfc_partition_static")
        torch.cuda.synchronize(cuda)
        assert torch.equal(c, b)
        # "allocates nothing": the free device memory is the same before and after two more calls
        big = torch.empty(max_atoms, dtype=torch.int64, device=cuda)
        torch.cuda.synchronize(cuda)
        free0, _ = torch.cuda.mem_get_info(cuda)
        for _ in range(2):
            _lib.check(L.dynb_sfc_partition_static(pos1.data_ptr(), max_atoms, None, 8, 0, big.data_ptr(), None, st),
                       "sfc_partition_static")
        torch.cuda.synchronize(cuda)
        free1, _ = torch.cuda.mem_get_info(cuda)
        assert free1 == free0, (free0, free1)
        # larger than the limit: refused with a clear message, nothing launched
        pos3 = torch.zeros(max_atoms + 1, 3, device=cuda)
        out = torch.empty(max_atoms + 1, dtype=torch.int64, device=cuda)
        rc = L.dynb_sfc_partition_static(pos3.data_ptr(), max_atoms + 1, None, 4, 0, out.data_ptr(), None,
                                         torch.cuda.current_stream(cuda).cuda_stream)
        assert rc == -1 and b"exceeds the built-in scratch" in L.dynb_last_error()
