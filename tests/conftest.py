import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle

    _oracle.build()
    return _oracle


@pytest.fixture(scope="session")
def ops():
    """The product ops; importing them requires the built CUDA library and, to call them, a GPU."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from rexsc_b200 import ops as _ops

    return _ops
