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
    """Launches on the stream torch uses: the tests build operands and fill result buffers
    with torch ops, and stream order is what makes a kernel see them (the context's own
    stream is non-blocking and would need explicit synchronisation on both sides). That
    stream is a created one, made torch's current stream for the whole session, because the
    legacy default stream cannot be captured into a CUDA graph."""
    import torch

    from lighthouse_b200.context import CudaContext

    stream = torch.cuda.Stream(device=0)
    torch.cuda.set_stream(stream)
    c = CudaContext(0, use_torch_stream=True)
    yield c
    torch.cuda.synchronize()
    c.close()


@pytest.fixture()
def own_stream_ctx(native_lib):
    """A context on its own non-blocking stream; the caller synchronises around its calls."""
    from lighthouse_b200.context import CudaContext

    c = CudaContext(0)
    yield c
    c.close()
