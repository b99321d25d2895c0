"""Split atoms of the distributed repartition (dynamis_b200.migrate.select_split_atoms) on CPU tensors: W emulated
ranks run the selection in lockstep (threads; the collective is a sum over the ranks' tensors) and must all get
the split atoms of the gathered, sorted (key, id) list — equal counts (reference closed form,
dynamis_state/src/csrc/partition/sfc_kernels.cu:114-137) and the weighted cut floor(cumsum * W / total)
(:139-173)."""

import threading

import numpy as np
import pytest
import torch

from dynamis_b200.migrate import select_split_atoms, split_positions


class _LockstepColl:
    """all_reduce(SUM) over W threads that call it in the same order."""

    def __init__(self, W):
        self.W = W
        self.slots = [None] * W
        self.barrier = threading.Barrier(W)
        self.local = threading.local()

    def bind(self, rank):
        self.local.rank = rank

    def all_reduce(self, t, op=None):
        self.slots[self.local.rank] = t
        self.barrier.wait()
        total = torch.stack(self.slots).sum(dim=0)
        self.barrier.wait()
        return total


def _run(W, keys, ids, owner, key_bits, id_bits, weights=None):
    N = keys.shape[0]
    coll = _LockstepColl(W)
    out = [None] * W
    err = []
    thr = None
    if weights is not None:
        total = int(weights.sum())
        thr = torch.tensor([max(1, ((s + 1) * total + W - 1) // W) for s in range(W - 1)], dtype=torch.int64)

    def work(rank):
        try:
            coll.bind(rank)
            mine = np.nonzero(owner == rank)[0]
            order = mine[np.lexsort((ids[mine], keys[mine]))]
            sk, sg = torch.from_numpy(keys[order]), torch.from_numpy(ids[order])
            if weights is None:
                out[rank] = select_split_atoms(coll, sk, sg, split_positions(N, W), key_bits, id_bits)
            else:
                out[rank] = select_split_atoms(coll, sk, sg, None, key_bits, id_bits, sw=torch.from_numpy(weights[order]), thresholds=thr)
        except Exception as e:  # a failing rank must not leave the others at the barrier for ever
            err.append(e)
            coll.barrier.abort()

    ts = [threading.Thread(target=work, args=(r,)) for r in range(W)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=120)
    assert not err, err
    return out


def _expected(W, keys, ids, weights=None):
    order = np.lexsort((ids, keys))
    N = keys.shape[0]
    if weights is None:
        at = np.asarray(split_positions(N, W))
    else:
        cs = np.cumsum(weights[order])
        total = int(cs[-1])
        at = np.asarray([int(np.searchsorted(cs, max(1, ((s + 1) * total + W - 1) // W), side="left")) for s in range(W - 1)])
        # the same cut as the reference's labels: label >= s + 1 from that atom on
        lab = np.minimum(cs * W // total, W - 1)
        for s in range(W - 1):
            first = int(np.argmax(lab >= s + 1)) if (lab >= s + 1).any() else N
            assert first == at[s]
    return keys[order][at], ids[order][at]


@pytest.mark.parametrize("W", [2, 3, 4, 8])
@pytest.mark.parametrize("key_range", [7, 1 << 20, (1 << 62) - 1])
def test_split_atoms_equal_counts_and_weighted(W, key_range):
    rng = np.random.default_rng(W * 1000 + (key_range % 97))
    N = 5000 + 17 * W
    keys = rng.integers(0, key_range + 1, N, dtype=np.int64)
    ids = rng.permutation(N).astype(np.int64)
    owner = rng.integers(0, W, N)
    owner[owner == W - 1] = 0 if W > 2 else owner[owner == W - 1]      # W > 2: the last rank holds nothing
    key_bits = max(1, int(key_range).bit_length())
    id_bits = max(1, (N - 1).bit_length())
    K, G = _expected(W, keys, ids)
    for k, g in _run(W, keys, ids, owner, key_bits, id_bits):
        assert np.array_equal(k.numpy(), K) and np.array_equal(g.numpy(), G)
    weights = rng.integers(0, 90, N, dtype=np.int64)
    weights[rng.integers(0, N, N // 10)] = 0                            # atoms without neighbours
    weights[rng.integers(0, N, 3)] = 40_000                              # a few atoms that cross several thresholds at once
    K, G = _expected(W, keys, ids, weights)
    for k, g in _run(W, keys, ids, owner, key_bits, id_bits, weights):
        assert np.array_equal(k.numpy(), K) and np.array_equal(g.numpy(), G)


# ------------------------------------------------------------------ the same over a real process group (gloo, 2 ranks)

_GLOO_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from dynamis_b200.migrate import _Coll, select_split_atoms, split_positions
rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
coll = _Coll()
assert coll.host and coll.W == W and coll.rank == rank
rng = np.random.default_rng(11)                       # the same stream on every rank: all know the whole system
N = 3001
keys = rng.integers(0, 1 << 30, N, dtype=np.int64); keys[rng.integers(0, N, N // 3)] = 12345      # a third of the keys tie
ids = rng.permutation(N).astype(np.int64)
weights = rng.integers(0, 50, N, dtype=np.int64)
owner = rng.integers(0, W, N)
mine = np.nonzero(owner == rank)[0]
order = mine[np.lexsort((ids[mine], keys[mine]))]
sk, sg, sw = torch.from_numpy(keys[order]), torch.from_numpy(ids[order]), torch.from_numpy(weights[order])
gorder = np.lexsort((ids, keys))
# equal counts
K, G = select_split_atoms(coll, sk, sg, split_positions(N, W), 30, 12)
at = np.asarray(split_positions(N, W))
assert np.array_equal(K.numpy(), keys[gorder][at]) and np.array_equal(G.numpy(), ids[gorder][at])
# weighted
total = int(coll.all_reduce(sw.sum().reshape(1).clone())[0]); assert total == int(weights.sum())
thr = torch.tensor([max(1, ((s + 1) * total + W - 1) // W) for s in range(W - 1)], dtype=torch.int64)
K, G = select_split_atoms(coll, sk, sg, None, 30, 12, sw=sw, thresholds=thr)
cs = np.cumsum(weights[gorder]); at = np.searchsorted(cs, thr.numpy(), side="left")
assert np.array_equal(K.numpy(), keys[gorder][at]) and np.array_equal(G.numpy(), ids[gorder][at])
# the row exchange of the migration: every rank sends rank-tagged rows, grouped by destination
send_counts = [3 + rank, 5 - rank][:W]
recv_counts = coll.exchange_counts(send_counts)
assert recv_counts == [[3, 4], [5, 4]][rank]
rows = torch.arange(sum(send_counts) * 2, dtype=torch.float32).reshape(-1, 2) + 100 * rank
got = coll.all_to_all_rows(rows, send_counts, recv_counts)
want = []
for p in range(W):
    pc = [3 + p, 5 - p]
    base = torch.arange(sum(pc) * 2, dtype=torch.float32).reshape(-1, 2) + 100 * p
    start = sum(pc[:rank]); want.append(base[start:start + pc[rank]])
assert torch.equal(got, torch.cat(want))
box = coll.all_gather(torch.tensor([float(rank), 2.0]))
assert box.shape == (W, 2) and box[:, 0].tolist() == [0.0, 1.0]
dist.barrier(); dist.destroy_process_group()
'''


def test_split_selection_and_row_exchange_over_gloo_world_size_2(tmp_path):
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29617", str(script), root]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
