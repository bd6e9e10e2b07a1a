"""Test configuration: the `gpu` marker, and the repository root on sys.path.

`-m "not gpu"` covers the oracle against the reference's known answers, the host logic and the C ABI's
symbols; `-m gpu` holds the parity tests proper, which call the CUDA kernels through the C ABI on a B200.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an sm_100 GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native():
    """The built C-ABI library (built on demand where nvcc exists)."""
    from tilejax_b200 import _lib

    if not _lib.LIBRARY.exists():
        from tilejax_b200.csrc.build import build

        build()
    return _lib.library()
