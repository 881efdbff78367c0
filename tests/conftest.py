import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    # Build whatever is missing or older than its sources.
    from oracle import build as oracle_build
    oracle_build.build()
    from yaxus_b200 import build as lib_build
    lib_build.build()


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def backend():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from yaxus_b200 import CudaBackend
    b = CudaBackend(0)
    yield b
    b.close()


@pytest.fixture(autouse=True)
def _clean_backend_error(request):
    yield
    if "backend" in request.fixturenames:
        try:
            b = request.getfixturevalue("backend")
            b.clear_error()
        except Exception:
            pass
