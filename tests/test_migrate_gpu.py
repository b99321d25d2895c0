"""Repartition + migration + halo rebuild on distributed state (no rank holds all atoms) against the
oracle's partition and halo maps of the gathered system; W = 2 and 4 ranks.  With fewer GPUs than ranks
the ranks share one GPU and use gloo for the (host-side) collectives."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("nproc", [2, 4])
def test_distributed_repartition_matches_gathered_partition(nproc):
    if not torch.cuda.is_available():
        pytest.skip("CUDA not available")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29560 + nproc), os.path.join(ROOT, "tests", "_migrate_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
