"""The device memory manager's protocol (lighthouse/execution/memory_manager.py:20-188 of the
reference) against a fake engine whose "device" is host memory: allocation by name, copies in
both directions, clone-and-free, and the errors."""

import ctypes

import numpy as np
import pytest

from lighthouse_b200.execution.memory_manager import CudaMemoryManager, ExternalMemoryManager, GPUMemoryManager, TorchCudaMemoryManager


class FakeEngine:
    def __init__(self):
        self.live, self.syncs = {}, 0

    def malloc(self, nbytes):
        buf = ctypes.create_string_buffer(max(nbytes, 1))
        self.live[ctypes.addressof(buf)] = buf
        return ctypes.addressof(buf)

    def free(self, ptr):
        del self.live[ptr]

    def memcpy_h2d(self, dst, src, nbytes):
        ctypes.memmove(dst, src, nbytes)

    def memcpy_d2h(self, dst, src, nbytes):
        ctypes.memmove(dst, src, nbytes)

    def sync(self):
        self.syncs += 1


def test_clone_copy_and_free():
    eng = FakeEngine()
    mm = GPUMemoryManager(eng)
    assert GPUMemoryManager is CudaMemoryManager
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    with mm.clone_host_buffers([a, a.T], names=["x", "y"]) as (dx, dy):  # a.T: non-contiguous source is staged
        assert mm.get("x") is dx and len(eng.live) == 2
        assert list(dx.shape) == [3, 4] and list(dx.strides) == [4, 1] and list(dy.shape) == [4, 3]
        back = np.zeros((4, 3), np.float32)
        mm.copy(dy, back)
        assert np.array_equal(back, a.T)
        with pytest.raises(ValueError, match="At least one of src or dst"):
            mm.copy(dx, dy)
        with pytest.raises(ValueError, match="size mismatch"):
            mm.copy(np.zeros(5, np.float32), dx)
        with pytest.raises(ValueError, match="C-contiguous"):
            mm.copy(dx, np.zeros((4, 3), np.float32).T)
        with pytest.raises(AssertionError, match="already exists"):
            mm.alloc((2,), "f32", name="x")
    assert not eng.live and eng.syncs == 2  # everything freed when the block ends
    with pytest.raises(AssertionError, match="No buffer found"):
        mm.get("x")
    d = mm.alloc((5,), np.float32)
    assert mm.get("buffer_0") is d
    mm.deallocate_all()
    assert not eng.live


def test_external_managers_do_not_allocate():
    mm = TorchCudaMemoryManager()
    assert isinstance(mm, ExternalMemoryManager)
    for call in (lambda: mm.alloc("x"), lambda: mm.get("x"), mm.deallocate_all):
        with pytest.raises(NotImplementedError):
            call()
    import torch

    with pytest.raises(ValueError, match="CUDA tensors"):
        with mm.get_memrefs([torch.zeros(2, 2)]):
            pass
