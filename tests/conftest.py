import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_addoption(parser):
    parser.addoption("--fake-device", action="store_true",
                     help="check the GPU tests themselves on a machine without a GPU: the context "
                          "is replaced by a CPU stand-in built on the oracle (tests/_fake.py)")
    parser.addoption("--emulated-device", action="store_true",
                     help="run the GPU tests without a GPU against the library's own code, compiled "
                          "as host code around stand-ins for the hardware (tests/_emulated.py); slow")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    if config.getoption("--fake-device"):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        import _fake
        _fake.install()
    if config.getoption("--emulated-device"):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        import _emulated
        _emulated.install()


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.binding import Reference
    return Reference()


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_host.npz")
    return dict(np.load(path))
