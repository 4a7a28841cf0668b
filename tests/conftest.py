"""Shared fixtures.  CPU tests (`-m "not gpu"`) check the oracle, the host logic and that the
C-ABI library loads; GPU tests (`-m gpu`) are the parity tests and call through the C ABI."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def ob():
    """The ctypes binding; builds the library first when nvcc is available and it is stale."""
    import shutil
    if shutil.which("nvcc"):
        from onellm_b200 import build as _b
        _b.build()
    import onellm_b200
    onellm_b200.lib()
    return onellm_b200


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("test marked gpu but no CUDA device is visible")
    torch.cuda.set_device(0)
    return torch


def rel_err(got, ref):
    """max |got - ref| / max |ref|: the norm every tolerance in these tests refers to."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(got - ref)) / max(float(np.max(np.abs(ref))), 1e-30))


class _DevicePointer:
    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr), False), "version": 2}


def device_view(torch, ptr, n, typestr="<f2"):
    """A torch tensor over `n` elements of device memory the library owns (e.g. the engine's KV cache)."""
    return torch.as_tensor(_DevicePointer(ptr, n, typestr), device="cuda")
