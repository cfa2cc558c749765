import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.cpu_oracle import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def lib():
    """The C-ABI shared library, loaded through the package's ctypes binding."""
    import infr_b200

    return infr_b200.load_library()


@pytest.fixture(scope="session")
def backend():
    import torch  # noqa: F401  (only for the availability probe below)

    import infr_b200

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    be = infr_b200.CudaBackend(device=0)
    yield be
    be.close()
