import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("CUDA not available")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def ref_ops():
    """torch.ops.dynamis_ref (the reference's own CUDA kernels, built by oracle/build_ref.py), or skip."""
    import torch

    from oracle import build_ref

    if not torch.cuda.is_available():
        pytest.skip("CUDA not available")
    if not build_ref.load():
        pytest.skip("oracle/_ref was not built")
    return torch.ops.dynamis_ref
