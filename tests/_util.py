"""Helpers shared by the test modules."""

from __future__ import annotations

import numpy as np
import torch

from oracle import cpu_oracle as O


def canon_t(edge_index: torch.Tensor, shifts: torch.Tensor) -> np.ndarray:
    ei = edge_index.detach().cpu().numpy()
    return O.canonical_edges(ei[0], ei[1], shifts.detach().cpu().numpy())


def canon_o(g: dict) -> np.ndarray:
    return O.canonical_edges(g["src"], g["dst"], g["shift"])


def digest_t(edge_index: torch.Tensor, shifts: torch.Tensor):
    """Order-independent digest of an edge set, computed on the tensor's device.  Same formula as
    oracle.cpu_oracle.edge_set_digest (int64 arithmetic wraps modulo 2^64 like uint64)."""
    src, dst = edge_index[0], edge_index[1]
    sh = shifts.round().to(torch.int64) + 512
    h = src * (-7046029254386353131) + dst * (-4417276706812531889)  # 0x9E37..15, 0xC2B2..4F as int64
    h = h ^ ((sh[:, 0] << 40) | (sh[:, 1] << 20) | sh[:, 2])
    h = h * (-2960836687051489901)  # 0xD6E8FEB86659FD93
    h = h ^ ((h >> 32) & 0xFFFFFFFF)
    total = int(h.sum().item()) & 0xFFFFFFFFFFFFFFFF
    return int(src.numel()), total


def assert_same_edges(a: np.ndarray, b: np.ndarray, what: str = ""):
    assert a.shape == b.shape, f"{what}: edge count {a.shape[0]} vs {b.shape[0]}"
    if a.shape[0]:
        bad = np.nonzero((a != b).any(axis=1))[0]
        assert bad.size == 0, f"{what}: first mismatch at row {bad[0]}: {a[bad[0]]} vs {b[bad[0]]}"
