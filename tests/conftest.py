import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs the CUDA path through the C ABI)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_cases.npz"))


@pytest.fixture(scope="session")
def rt():
    """The runtime library, initialised on device 0 with launches routed to torch's current stream."""
    import torch

    from docc_b200 import _lib, ops

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    ops.init(0)
    ops.set_stream(torch.cuda.current_stream().cuda_stream)
    return _lib.lib()


def relerr(got, ref):
    """Norm-wise relative error max|got-ref| / max|ref| (BLAS builds differ in summation order)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.max(np.abs(ref)) if ref.size else 1.0
    if denom == 0:
        denom = 1.0
    return float(np.max(np.abs(got - ref)) / denom) if ref.size else 0.0
