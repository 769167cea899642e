"""Test configuration: the ``gpu`` marker and the import path.

``-m "not gpu"`` runs everywhere (oracle vs golden vectors, host logic, C-ABI symbol checks);
``-m gpu`` needs a B200 and calls the CUDA kernels through the C ABI.
"""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU; runs the CUDA kernels through the C ABI")


@pytest.fixture(scope="session")
def native_lib():
    """The built native library (builds it on first use; never falls back to anything else)."""
    from aster_b200 import build, _native

    build.build()
    return _native.lib()


@pytest.fixture(scope="session")
def gpu(native_lib):
    """Initialises device 0 and fails loudly when the GPU or the library is not usable."""
    from aster_b200 import _native as nat

    nat.call("b200_init", 0)
    props = nat.device_props(0)
    assert props.cc_major == 10, f"expected an sm_100 device, found {props.name!r} cc {props.cc_major}.{props.cc_minor}"
    return props


@pytest.fixture(scope="session")
def golden():
    import json

    with open(os.path.join(ROOT, "tests", "golden", "reference_golden.json")) as f:
        return json.load(f)
