import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def ctx():
    """One CUDA context for the whole GPU session (fails loudly without the library)."""
    from ullm_b200 import backend

    c = backend.CudaContext(0)
    yield c
    c.close()
