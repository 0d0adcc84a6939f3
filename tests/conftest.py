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
    """The CPU checkers (plain-C port and, where built, the compiled reference bodies)."""
    import oracle as O
    O.port_lib()
    return O


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import _lib
    _lib.lib()  # fail loudly if the extension is missing
    return jg
