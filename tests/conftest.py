import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "fake_comfy")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    """The package directory imported as `feather_b200`."""
    import __graft_entry__

    return __graft_entry__.load_package()


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"), allow_pickle=False)


@pytest.fixture(scope="session")
def native(pkg):
    import importlib

    return importlib.import_module("feather_b200.kernel.b200.native")


@pytest.fixture(scope="session")
def hip_kernel(pkg):
    import importlib

    return importlib.import_module("feather_b200.kernel.hip.hip_kernel")


@pytest.fixture(scope="session")
def cuda_dev():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
