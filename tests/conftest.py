import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def backend():
    """One CudaBackend on cuda:0 for the whole session.  No fallback: a missing library or
    device fails the GPU tests loudly."""
    from moe4all_b200 import build as _build
    from moe4all_b200 import CudaBackend

    _build.build()
    be = CudaBackend(0)
    yield be
    be.close()
