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
    """The plain-C CPU restatement of the libpymo arithmetic (test infrastructure)."""
    from oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU code compiled into oracle/_ref (only where it was built)."""
    from oracle import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libaimet_ref.so not built (needs the reference checkout)")
    return Reference()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
