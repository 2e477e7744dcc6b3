"""Shared pytest configuration.

``-m "not gpu"`` tests run anywhere (oracle vs golden vectors, host logic, symbol exports);
``-m gpu`` tests are the parity tests proper: they call the CUDA kernels through the C ABI
and compare against the CPU oracle.
"""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")
PAYLOADS = os.path.join(ROOT, "tests", "payloads")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs the CUDA kernels through the C ABI)")


@pytest.fixture(scope="session")
def native_lib():
    """The built shared library; built on demand where nvcc exists."""
    from lighthouse_b200 import _native
    from lighthouse_b200.build import build

    if not _native.lib_path().exists():
        build()
    return _native.load()


@pytest.fixture(scope="session")
def ctx(native_lib):
    from lighthouse_b200.context import CudaContext

    c = CudaContext(0)
    yield c
    c.close()
