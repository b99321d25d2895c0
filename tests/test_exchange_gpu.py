"""GPU tests of the halo-exchange kernels on ONE GPU.

Pack: the reference's dynamis_model/tests/test_push_buffer.py cases (basic, duplicates, single row,
identity, reversed, F in {4, 10, 16, 64, 65, 128, 256}, 100,000 rows, empty, validation text).
One-sided push: several ranks are driven from this one process (all pushes first, then all waits,
so that no kernel ever waits for work queued behind it); ghost rows must be bit-exact, reverse
accumulation within 1e-6 relative of the float64 oracle.  The reference's two-rank known answer
(dynamis_model/tests/test_ipc_exchange.py:33-59,138-207) is included.
"""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("F", [3, 4, 10, 16, 64, 65, 128, 256])
def test_pack_matches_index(cuda, F):
    for seed in range(5):
        g = torch.Generator(device="cpu").manual_seed(seed)
        inp = torch.randn(500, F, generator=g).to(cuda)
        for locs in (torch.randint(0, 500, (300,), generator=g), torch.tensor([7, 7, 7, 0, 499]), torch.tensor([3]),
                     torch.arange(500), torch.arange(499, -1, -1)):
            locs = locs.to(cuda)
            buf = torch.empty(locs.numel(), F, device=cuda)
            out = D.push_buffer_create(inp, buf, locs)
            assert out is buf and torch.equal(buf, inp[locs])


def test_pack_large_and_empty(cuda):
    for F in (64, 65):
        inp = torch.randn(100_000, F, device=cuda)
        locs = torch.randint(0, 100_000, (100_000,), device=cuda)
        buf = torch.empty(100_000, F, device=cuda)
        assert torch.equal(D.push_buffer_create(inp, buf, locs), inp[locs])
    buf = torch.empty(0, 8, device=cuda)
    assert D.push_buffer_create(torch.randn(4, 8, device=cuda), buf, torch.empty(0, dtype=torch.int64, device=cuda)).shape == (0, 8)


def test_pack_validation(cuda):
    inp, buf, locs = torch.randn(4, 8, device=cuda), torch.empty(2, 8, device=cuda), torch.tensor([0, 1], device=cuda)
    with pytest.raises(RuntimeError, match="input must be a CUDA tensor"):
        D.push_buffer_create(inp.cpu(), buf, locs)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        D.push_buffer_create(torch.randn(8, 4, device=cuda).t(), buf, locs)
    with pytest.raises(RuntimeError, match="input datatype must be float32"):
        D.push_buffer_create(inp.double(), buf, locs)
    with pytest.raises(RuntimeError, match="buffer datatype must be float32"):
        D.push_buffer_create(inp, buf.double(), locs)
    with pytest.raises(RuntimeError, match="input must have 2 dimensions"):
        D.push_buffer_create(inp.flatten(), buf, locs)
    with pytest.raises(RuntimeError, match="buffer must have 2 dimensions"):
        D.push_buffer_create(inp, buf.flatten(), locs)
    with pytest.raises(RuntimeError, match="input_locs must have 1 dimension"):
        D.push_buffer_create(inp, buf, locs.unsqueeze(0))
    with pytest.raises(RuntimeError, match="buffer rows must match size of input_locs"):
        D.push_buffer_create(inp, torch.empty(3, 8, device=cuda), locs)
    with pytest.raises(RuntimeError, match="input and buffer must have same number of columns"):
        D.push_buffer_create(inp, torch.empty(2, 4, device=cuda), locs)
    with pytest.raises(RuntimeError, match="input_locs datatype must be int64"):
        D.push_buffer_create(inp, buf, locs.int())


def _make_ranks(plans, F, dev, dtype=torch.float32, wait_ns=5_000_000_000):
    """plans[r] = (send_offsets, send_local, recv_offsets, n_local) as numpy / ints."""
    W = len(plans)
    ex = [D.FeatureExchanger(wait_ns) for _ in range(W)]
    metas = [ex[r].local_setup(torch.as_tensor(p[0]), torch.as_tensor(p[1]), torch.as_tensor(p[2]), p[3], F, r, W, dev, dtype)
             for r, p in enumerate(plans)]
    for e in ex:
        e.connect(metas)
    return ex


def _exchange_all(ex, feats):
    pend = [e.forward_begin(f) for e, f in zip(ex, feats)]
    return [e.forward_end(o, g) for e, (o, g) in zip(ex, pend)]


def _exchange_back_all(ex, grads):
    pend = [e.backward_begin(g) for e, g in zip(ex, grads)]
    return [e.backward_end(g, gen) for e, (g, gen) in zip(ex, pend)]


def test_two_rank_known_answer(cuda):
    # rank 0 owns 10 atoms and sends [0,2,4,6,8]; rank 1 owns 12 and sends [1,3,5,7,9,11]
    p0 = (np.array([0, 0, 5]), np.array([0, 2, 4, 6, 8]), np.array([0, 0, 6]), 10)
    p1 = (np.array([0, 6, 6]), np.array([1, 3, 5, 7, 9, 11]), np.array([0, 5, 5]), 12)
    F = 4
    ex = _make_ranks([p0, p1], F, cuda)
    feats = [(torch.arange(n, device=cuda, dtype=torch.float32) + r * 1000).unsqueeze(1).repeat(1, F).contiguous()
             for r, n in enumerate((10, 12))]
    out = _exchange_all(ex, feats)
    assert out[0].shape == (16, F) and out[1].shape == (17, F)
    assert out[0][10:, 0].tolist() == [1001.0, 1003.0, 1005.0, 1007.0, 1009.0, 1011.0]
    assert out[1][12:, 0].tolist() == [0.0, 2.0, 4.0, 6.0, 8.0]
    back = _exchange_back_all(ex, [torch.ones_like(o) for o in out])
    assert back[0][:, 0].tolist() == [2.0, 1.0] * 5
    assert back[1][:, 0].tolist() == [1.0, 2.0] * 6
    for e in ex:
        e.check_status()
        e.teardown()


@pytest.mark.parametrize("W,F,dtype", [(3, 3, torch.float32), (4, 128, torch.float32), (8, 128, torch.float32), (3, 5, torch.float64)])
def test_emulated_ranks_match_oracle(cuda, W, F, dtype):
    rng = np.random.default_rng(W * 100 + F)
    n, L = 6000, 44.0
    pos = (rng.random((n, 3)) * L).astype(np.float32)
    cell = (np.eye(3) * L).astype(np.float32)
    g = O.radius_graph(pos, cell, [1, 1, 1], np.float32(6.5))
    pid = O.sfc_partition(pos, None, W, 0)
    maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
    plans = [(m["send_offsets"], m["send_local_indices"], m["recv_offsets"], m["num_local"]) for m in maps]
    ex = _make_ranks(plans, F, cuda, dtype)
    npdt = np.float32 if dtype == torch.float32 else np.float64
    feats_np = [rng.standard_normal((m["num_local"], F)).astype(npdt) for m in maps]
    so = [m["send_offsets"] for m in maps]
    sl = [m["send_local_indices"] for m in maps]
    ro = [m["recv_offsets"] for m in maps]
    nl = [m["num_local"] for m in maps]
    for it in range(3):  # several generations: exercises the parity double buffering
        feats_it = [f + it for f in feats_np]
        out = _exchange_all(ex, [torch.as_tensor(f, device=cuda) for f in feats_it])
        ref = O.exchange_forward(feats_it, so, sl, ro)
        for r in range(W):
            np.testing.assert_array_equal(out[r].cpu().numpy(), ref[r])  # payload copies are bit-exact
        grads_np = [rng.standard_normal(o.shape).astype(npdt) for o in ref]
        back = _exchange_back_all(ex, [torch.as_tensor(x, device=cuda) for x in grads_np])
        refb = O.exchange_backward(grads_np, nl, so, sl, ro)
        for r in range(W):
            np.testing.assert_allclose(back[r].cpu().numpy(), refb[r], rtol=1e-6 if dtype == torch.float32 else 1e-12,
                                       atol=1e-6 if dtype == torch.float32 else 1e-12)
        # deterministic: a second identical backward gives identical bits
        back2 = _exchange_back_all(ex, [torch.as_tensor(x, device=cuda) for x in grads_np])
        for r in range(W):
            assert torch.equal(back[r], back2[r])
    for e in ex:
        e.check_status()
        e.teardown()


def test_wait_budget_expires_with_status_not_a_hang(cuda):
    """A peer that never signals: the bounded wait runs out after its budget, sets the status words,
    and the context stays usable.  The library path reports it by itself: the next push raises
    without anybody calling check_status, and the exchanger stays unusable until it is set up again."""
    p0 = (np.array([0, 0, 2]), np.array([0, 1]), np.array([0, 0, 2]), 4)
    p1 = (np.array([0, 2, 2]), np.array([0, 1]), np.array([0, 2, 2]), 4)
    ex = _make_ranks([p0, p1], 4, cuda, wait_ns=2_000_000)  # 2 ms
    x = torch.randn(4, 4, device=cuda)
    out, gen = ex[0].forward_begin(x)       # rank 1 never pushes
    ex[0].forward_end(out, gen)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="timed out"):
        ex[0].feature_push_forward(x)       # no check_status(): the push itself notices
    with pytest.raises(RuntimeError, match="set up again"):
        ex[0].feature_push_backward(torch.zeros(6, 4, device=cuda))
    with pytest.raises(RuntimeError, match="timed out"):
        ex[0].check_status()
    assert torch.equal(x + 0, x)  # the device still works
    for e in ex:
        e.teardown()


def test_drift_word_rides_on_every_handshake(cuda):
    """Every signal carries the rank's drift word; after every wait each rank holds the OR over all
    ranks (the scheme of the reference's dynamis/tests/test_drift_watchdog.py:97-120), forward and
    reverse, over 50 generations with random words."""
    W, F = 4, 8
    rng = np.random.default_rng(5)
    n, L = 3000, 36.0
    pos = (rng.random((n, 3)) * L).astype(np.float32)
    g = O.radius_graph(pos, (np.eye(3) * L).astype(np.float32), [1, 1, 1], np.float32(6.5))
    pid = O.sfc_partition(pos, None, W, 0)
    maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
    plans = [(m["send_offsets"], m["send_local_indices"], m["recv_offsets"], m["num_local"]) for m in maps]
    ex = _make_ranks(plans, F, cuda)
    local = [torch.zeros(1, dtype=torch.int32, device=cuda) for _ in range(W)]
    glob = [torch.full((1,), -1, dtype=torch.int32, device=cuda) for _ in range(W)]
    for e, l, gl in zip(ex, local, glob):
        e.set_watchdog_flags(l, gl)
    feats = [torch.randn(m["num_local"], F, device=cuda) for m in maps]
    for it in range(50):
        words = rng.integers(0, 4, W) if it % 5 else np.zeros(W, dtype=np.int64)
        for l, w in zip(local, words):
            l.fill_(int(w))
        out = _exchange_all(ex, feats)
        want = int(np.bitwise_or.reduce(words))
        assert [int(x.item()) for x in glob] == [want] * W, f"forward generation {it}"
        words2 = rng.integers(0, 4, W)
        for l, w in zip(local, words2):
            l.fill_(int(w))
        _exchange_back_all(ex, [torch.ones_like(o) for o in out])
        assert [int(x.item()) for x in glob] == [int(np.bitwise_or.reduce(words2))] * W, f"reverse generation {it}"
    ex[1].clear_watchdog_flags()     # a rank that stops carrying the flag contributes 0 and leaves its own word alone
    glob[1].fill_(77)
    for l in local:
        l.fill_(1)
    local[1].fill_(2)
    _exchange_all(ex, feats)
    assert [int(x.item()) for x in glob] == [1, 77, 1, 1]
    with pytest.raises(RuntimeError, match="int32"):
        ex[0].set_watchdog_flags(torch.zeros(1, device=cuda), glob[0])
    for e in ex:
        e.check_status()
        e.teardown()


def test_results_live_in_peer_visible_slots_and_fall_back_when_held(cuda):
    """From the second generation on the ghost rows land in the result tensor itself (a slot of the
    exchange allocation).  A caller that keeps every result alive exhausts the ring; the exchange then
    goes through the staging buffer and must still be right, and earlier results must stay intact."""
    W, F = 3, 16
    rng = np.random.default_rng(11)
    n, L = 4000, 40.0
    pos = (rng.random((n, 3)) * L).astype(np.float32)
    g = O.radius_graph(pos, (np.eye(3) * L).astype(np.float32), [1, 1, 1], np.float32(6.5))
    pid = O.sfc_partition(pos, None, W, 0)
    maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
    plans = [(m["send_offsets"], m["send_local_indices"], m["recv_offsets"], m["num_local"]) for m in maps]
    so, sl, ro = [m["send_offsets"] for m in maps], [m["send_local_indices"] for m in maps], [m["recv_offsets"] for m in maps]
    ex = _make_ranks(plans, F, cuda)

    def inside(e, t):
        return e._alloc.ptr <= t.data_ptr() < e._alloc.ptr + e.layout["stage_off"][0]

    held, refs = [], []
    for it in range(8):
        feats = [rng.standard_normal((m["num_local"], F)).astype(np.float32) for m in maps]
        out = _exchange_all(ex, [torch.as_tensor(f, device=cuda) for f in feats])
        ref = O.exchange_forward(feats, so, sl, ro)
        for r in range(W):
            np.testing.assert_array_equal(out[r].cpu().numpy(), ref[r])
        if it == 0:
            assert not any(inside(e, o) for e, o in zip(ex, out))     # nothing was announced before the first signal
        elif it < 4:
            assert all(inside(e, o) for e, o in zip(ex, out)), it      # ring of 3 slots
        held.append(out)
        refs.append(ref)
        if it >= 4:
            # ring exhausted by the results still held: staging path, and nothing held was overwritten
            assert not any(inside(e, o) for e, o in zip(ex, out)), it
        for o_old, r_old in zip(held, refs):
            for r in range(W):
                np.testing.assert_array_equal(o_old[r].cpu().numpy(), r_old[r])
    del held, out, o_old
    for it in range(3):  # slots are free again once the tensors are gone
        feats = [rng.standard_normal((m["num_local"], F)).astype(np.float32) for m in maps]
        out = _exchange_all(ex, [torch.as_tensor(f, device=cuda) for f in feats])
        ref = O.exchange_forward(feats, so, sl, ro)
        for r in range(W):
            np.testing.assert_array_equal(out[r].cpu().numpy(), ref[r])
        if it >= 1:
            assert all(inside(e, o) for e, o in zip(ex, out))
        del out
    for e in ex:
        e.check_status()
        e.teardown()


@pytest.mark.parametrize("ring", [0, 3])
def test_copy_engine_variant_matches(cuda, ring):
    """set_ce_threshold_bytes: pack + one peer copy per rank instead of SM stores (reference:
    ipc_exchanger.cpp:526-569); same rows."""
    W, F = 3, 32
    rng = np.random.default_rng(21)
    n, L = 3000, 36.0
    pos = (rng.random((n, 3)) * L).astype(np.float32)
    g = O.radius_graph(pos, (np.eye(3) * L).astype(np.float32), [1, 1, 1], np.float32(6.5))
    pid = O.sfc_partition(pos, None, W, 0)
    maps = [O.build_halo_maps(g["src"], g["dst"], pid, r, W) for r in range(W)]
    plans = [(m["send_offsets"], m["send_local_indices"], m["recv_offsets"], m["num_local"]) for m in maps]
    so, sl, ro = [m["send_offsets"] for m in maps], [m["send_local_indices"] for m in maps], [m["recv_offsets"] for m in maps]
    ex = [D.FeatureExchanger(5_000_000_000, result_ring=ring) for _ in range(W)]
    metas = [ex[r].local_setup(torch.as_tensor(p[0]), torch.as_tensor(p[1]), torch.as_tensor(p[2]), p[3], F, r, W, cuda)
             for r, p in enumerate(plans)]
    for e in ex:
        e.connect(metas)
        e.set_ce_threshold_bytes(1)
        assert e.ce_threshold_bytes() == 1
    for it in range(3):
        feats = [rng.standard_normal((m["num_local"], F)).astype(np.float32) for m in maps]
        out = _exchange_all(ex, [torch.as_tensor(f, device=cuda) for f in feats])
        ref = O.exchange_forward(feats, so, sl, ro)
        for r in range(W):
            np.testing.assert_array_equal(out[r].cpu().numpy(), ref[r])
    for e in ex:
        e.check_status()
        e.teardown()


def test_new_halo_plan_keeps_the_allocation_while_it_fits(cuda):
    """local_setup with head-room: a second plan that fits keeps the exchange allocation (no new peer-visible
    memory, no new mappings), the generations start over and the exchange is right; a plan beyond the
    capacity allocates anew."""
    W, F = 3, 16
    rng = np.random.default_rng(31)

    def plans_for(n, L, r):
        pos = (rng.random((n, 3)) * L).astype(np.float32)
        g = O.radius_graph(pos, (np.eye(3) * L).astype(np.float32), [1, 1, 1], np.float32(r))
        pid = O.sfc_partition(pos, None, W, 0)
        return [O.build_halo_maps(g["src"], g["dst"], pid, k, W) for k in range(W)]

    def check(ex, maps):
        so, sl, ro = [m["send_offsets"] for m in maps], [m["send_local_indices"] for m in maps], [m["recv_offsets"] for m in maps]
        nl = [m["num_local"] for m in maps]
        for it in range(3):
            feats = [rng.standard_normal((m["num_local"], F)).astype(np.float32) for m in maps]
            out = _exchange_all(ex, [torch.as_tensor(f, device=cuda) for f in feats])
            ref = O.exchange_forward(feats, so, sl, ro)
            for k in range(W):
                np.testing.assert_array_equal(out[k].cpu().numpy(), ref[k])
            grads = [rng.standard_normal(o.shape).astype(np.float32) for o in ref]
            back = _exchange_back_all(ex, [torch.as_tensor(x, device=cuda) for x in grads])
            refb = O.exchange_backward(grads, nl, so, sl, ro)
            for k in range(W):
                np.testing.assert_allclose(back[k].cpu().numpy(), refb[k], rtol=1e-6, atol=1e-6)
            del out, back

    def setup(ex, maps):
        metas = [ex[k].local_setup(torch.as_tensor(m["send_offsets"]), torch.as_tensor(m["send_local_indices"]),
                                   torch.as_tensor(m["recv_offsets"]), m["num_local"], F, k, W, cuda, headroom=0.5)
                 for k, m in enumerate(maps)]
        for e in ex:
            e.connect(metas)

    ex = [D.FeatureExchanger(5_000_000_000) for _ in range(W)]
    a = plans_for(3000, 36.0, 6.5)
    setup(ex, a)
    ptrs = [e._alloc.ptr for e in ex]
    check(ex, a)
    b = plans_for(3300, 36.0, 6.0)           # other sizes, within the head-room
    setup(ex, b)
    assert [e._alloc.ptr for e in ex] == ptrs
    check(ex, b)
    c = plans_for(9000, 40.0, 6.5)           # beyond the capacity: new allocations
    setup(ex, c)
    check(ex, c)
    assert all(e.layout["capacity"][0] >= m["num_local"] + int(m["recv_offsets"][-1]) for e, m in zip(ex, c))
    for e in ex:
        e.check_status()
        e.teardown()


def test_push_rows_skips_and_reports_rows_out_of_range(cuda):
    """dynb_push_rows with a source index outside the input and a destination row beyond the target's
    capacity: both rows are skipped (nothing is written out of bounds) and the bad word is set."""
    import ctypes

    from dynamis_b200 import _lib

    L = _lib.lib()
    x = torch.arange(40, dtype=torch.float32, device=cuda).reshape(10, 4)
    dst = torch.full((6, 4), -1.0, device=cuda)
    guard = dst.clone()
    idx = torch.tensor([0, 3, 99, -1, 5], dtype=torch.int64, device=cuda)   # two bad source rows
    # one target: capacity 4 rows, rows start at row 0 -> logical row 4 would land on row 4 >= capacity
    table = torch.tensor([dst.data_ptr(), 0, 0, 5, 4], dtype=torch.int64, device=cuda)
    bad = torch.zeros(1, dtype=torch.int32, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    assert L.dynb_push_rows(x.data_ptr(), 10, 16, idx.data_ptr(), 0, table.data_ptr(), 1, 5, 16, bad.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 1
    assert torch.equal(dst[0], x[0]) and torch.equal(dst[1], x[3])
    assert torch.equal(dst[2:], guard[2:])


def test_backward_before_setup_raises(cuda):
    e = D.FeatureExchanger()
    with pytest.raises(RuntimeError, match="not set up"):
        e.feature_push_backward(torch.zeros(2, 2, device=cuda), (2, 2), None)
    g = D.GPUDirectExchanger()
    import torch.distributed as dist
    if not dist.is_initialized():
        with pytest.raises(RuntimeError, match="not setup for backward"):
            g.feature_push_backward(torch.zeros(2, 2, device=cuda), (2, 2), None)
