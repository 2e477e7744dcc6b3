"""Who owns the device buffers of a run.

The runner talks to a memory manager through the protocol of the reference
(lighthouse/execution/memory_manager.py:20-188): ``alloc`` / ``get`` / ``deallocate_all`` for a
manager that owns device memory, ``copy`` and ``clone_host_buffers`` on top of that for one
that moves host arrays, ``get_memrefs`` for one that only wraps buffers the caller already
holds. The reference's ``GPUMemoryManager`` reaches the device through ``gpu_alloc_*`` /
``gpu_copy_*`` / ``gpu_dealloc_*`` functions compiled into the payload; this backend has the
same three verbs in its library (``lh_b200_malloc`` / ``lh_b200_memcpy`` / ``lh_b200_free``),
so nothing is emitted into the payload and the "execution engine" handed to a manager is the
``CudaContext``.
"""

from __future__ import annotations

import abc
import ctypes
from contextlib import contextmanager
from dataclasses import dataclass, field

import numpy as np

from .._native import contiguous_strides
from ..utils.memref import make_descriptor
from ..utils.numpy import mlir_to_numpy_dtype, numpy_to_mlir_type


class MemoryManager(abc.ABC):
    """What every manager answers: named device buffers as memref descriptors."""

    @abc.abstractmethod
    def alloc(self, name: str | None = None, **kwargs) -> ctypes.Structure:
        """New device buffer; returns its descriptor."""

    @abc.abstractmethod
    def get(self, name: str) -> ctypes.Structure:
        """Descriptor of the buffer allocated under ``name``."""

    @abc.abstractmethod
    def deallocate_all(self):
        """Frees everything this manager allocated."""

    @staticmethod
    def emit_memory_management_funcs(payload_module, **kwargs):
        """Hook the reference uses to add its alloc / copy / dealloc helpers to the payload
        module; the library provides those here, so the payload is left as it is."""


@dataclass
class ExternalMemoryManager(MemoryManager, abc.ABC):
    """For buffers that already live on the device and belong to the caller: the manager
    only describes them (``get_memrefs``) and refuses to allocate."""

    execution_engine: object = None

    @abc.abstractmethod
    def get_memrefs(self, inputs):
        """Context manager yielding one descriptor per input."""

    def alloc(self, name: str | None = None, **kwargs) -> ctypes.Structure:
        raise NotImplementedError("Allocation not supported.")

    def get(self, name: str) -> ctypes.Structure:
        raise NotImplementedError("Lookup not supported.")

    def deallocate_all(self):
        raise NotImplementedError("Deallocation not supported.")


@dataclass
class DeviceMemoryManager(MemoryManager, abc.ABC):
    """A manager that owns device memory and moves host arrays in and out of it."""

    execution_engine: object = None

    @abc.abstractmethod
    def copy(self, src, dst):
        """Between a host array and a device buffer, in either direction."""

    @abc.abstractmethod
    def clone_host_buffers(self, host_inputs: list[np.ndarray], names: list[str] | None = None):
        """Context manager: device copies of the host arrays for the duration of the block."""


@dataclass
class _DeviceBuffer:
    descriptor: ctypes.Structure
    dtype: np.dtype
    nbytes: int


@dataclass
class CudaMemoryManager(DeviceMemoryManager):
    """``lh_b200_malloc`` for storage, ``lh_b200_memcpy`` for the traffic. A descriptor carries
    no element type or byte size, so both are remembered per buffer."""

    _buffers: dict[str, _DeviceBuffer] = field(default_factory=dict)
    _unnamed: int = 0

    def alloc(self, shape: tuple[int, ...], elem_type, name: str | None = None) -> ctypes.Structure:
        if name is None:
            name, self._unnamed = f"buffer_{self._unnamed}", self._unnamed + 1
        assert name not in self._buffers, f"Buffer with name '{name}' already exists."
        dtype = mlir_to_numpy_dtype(elem_type) if isinstance(elem_type, str) else np.dtype(elem_type)
        nbytes = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        descriptor = make_descriptor(self.execution_engine.malloc(nbytes), shape, contiguous_strides(shape))
        self._buffers[name] = _DeviceBuffer(descriptor, dtype, nbytes)
        return descriptor

    def get(self, name: str) -> ctypes.Structure:
        assert name in self._buffers, f"No buffer found with name '{name}'."
        return self._buffers[name].descriptor

    def deallocate_all(self):
        for buf in self._buffers.values():
            self.execution_engine.free(buf.descriptor.allocated)
        self._buffers.clear()
        self._unnamed = 0

    def _size_of(self, descriptor) -> int:
        for buf in self._buffers.values():
            if buf.descriptor is descriptor:
                return buf.nbytes
        raise ValueError("memref was not allocated by this manager")

    def copy(self, src, dst):
        host_src, host_dst = isinstance(src, np.ndarray), isinstance(dst, np.ndarray)
        if host_src and host_dst:
            np.copyto(dst, src)
        elif host_src:
            staged = np.ascontiguousarray(src)
            if staged.nbytes != self._size_of(dst):
                raise ValueError("size mismatch between host array and device buffer")
            self.execution_engine.memcpy_h2d(dst.allocated, staged.ctypes.data, staged.nbytes)
            self.execution_engine.sync()  # ``staged`` may be a temporary: finish before it goes away
        elif host_dst:
            if not (dst.flags["C_CONTIGUOUS"] and dst.flags["WRITEABLE"]):
                raise ValueError("destination host array must be C-contiguous and writeable")
            if dst.nbytes != self._size_of(src):
                raise ValueError("size mismatch between device buffer and host array")
            self.execution_engine.memcpy_d2h(dst.ctypes.data, src.allocated, dst.nbytes)
        else:
            raise ValueError("At least one of src or dst must be a numpy array.")

    @contextmanager
    def clone_host_buffers(self, host_inputs: list[np.ndarray], names: list[str] | None = None):
        try:
            clones = []
            for i, host in enumerate(host_inputs):
                clones.append(self.alloc(host.shape, numpy_to_mlir_type(host.dtype), name=names[i] if names is not None else None))
                self.copy(host, clones[-1])
            yield clones
        finally:
            self.deallocate_all()


# the reference's examples ask for ``GPUMemoryManager``; on this backend that is the CUDA one
GPUMemoryManager = CudaMemoryManager


class TorchCudaMemoryManager(ExternalMemoryManager):
    """CUDA ``torch.Tensor`` arguments by pointer, shape and strides - what
    ``TorchMemoryManager`` (lighthouse/ingress/torch/compile.py:42-48) does for the reference."""

    def __init__(self, execution_engine=None):
        self.execution_engine = execution_engine

    @contextmanager
    def get_memrefs(self, inputs):
        if not all(hasattr(t, "data_ptr") and t.is_cuda for t in inputs):
            raise ValueError("TorchCudaMemoryManager takes CUDA tensors")
        yield [make_descriptor(t.data_ptr(), tuple(t.shape), tuple(t.stride())) for t in inputs]
