import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_vectors.npz"))


@pytest.fixture(scope="session")
def port():
    """The C restatement of the reference's path (the checker)."""
    from oracle.loader import Port
    return Port()


@pytest.fixture(scope="session")
def ref():
    """The reference's own code, when its compiled form is present."""
    from oracle.loader import Ref, ref_available
    if not ref_available():
        pytest.skip("oracle/_ref/librpl_ref.so not built (reference tree absent)")
    return Ref()


@pytest.fixture(scope="session")
def lib():
    """librpl.so through ctypes; built first if this machine has nvcc and no copy yet."""
    from rpl_b200 import build, capi
    if not os.path.exists(capi.LIB_PATH):
        build.build()
    return capi.load()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def bits(a):
    """Bit pattern view for exact float comparison (distinguishes -0.0 and NaN payloads)."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a
