import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 for the GPU tests; building the library is part of the product
    path, so a missing .so is an error here, not a skip."""
    import torch

    import engine_b200

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    context = engine_b200.RibnContext(0)
    yield context
    context.synchronize()
    context.close()
