"""pytest configuration: the `gpu` marker and import paths.

`-m "not gpu"` runs here without a GPU: the oracle against the golden vectors, the
host-side logic (registry, planner/validation error codes, multi-rank sharding on
gloo) and the C-ABI export check.  `-m gpu` holds the parity tests proper; they call
the CUDA kernels through the C ABI and through torch.ops.pcie_through.
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def hfk():
    """The C-ABI library through ctypes; building it on demand when it is missing."""
    from heterofusedkernels_b200 import build, capi

    build.build_capi()
    return capi


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda", 0)
