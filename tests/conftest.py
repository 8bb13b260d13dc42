import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "ref_b200.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    if not os.path.exists(GOLDEN):
        pytest.skip("tests/golden/ref_b200.npz not generated yet")
    return dict(np.load(GOLDEN))


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def capi():
    """The product module, as a caller of the reference would import it."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import F2CGTLib
    return F2CGTLib
