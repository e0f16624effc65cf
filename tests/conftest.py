import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Both libraries exist before any test runs (nvcc and gcc work without a GPU)."""
    from mojolearn_b200.csrc import build as cuda_build
    from oracle import build as oracle_build
    cuda_build.build()
    oracle_build.build()
