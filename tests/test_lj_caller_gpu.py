"""A model written like the reference's LJ caller runs on the drop-in packages (``dynamis_state`` /
``dynamis_model`` resolved to dynamis_b200) and reproduces a dense float64 evaluation: on one rank, and —
where two GPUs are present — on two ranks with the positions, atom types and force gradients going
through the halo exchange (tolerances as dynamis/tests/test_simulation_regression.py:51-53)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("nproc", [1, 2])
def test_lj_caller_on_the_drop_in_packages(nproc):
    if not torch.cuda.is_available() or torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29540 + nproc), os.path.join(ROOT, "tests", "_lj_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
