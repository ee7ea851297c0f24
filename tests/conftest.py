"""pytest configuration: the ``gpu`` marker and shared fixtures.

Tests marked ``gpu`` need a B200 and go through the C ABI of libspio_b200; everything else
runs on a machine without a GPU (oracle against golden vectors, host logic, symbol export).
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """Build the native library and the C oracle if they are missing or stale."""
    from spio_b200 import build as native_build
    from oracle import oracle

    native_build.build()
    oracle.build()
