"""Memory managers with the protocol of lighthouse/execution/memory_manager.py:20-188.

The reference's ``GPUMemoryManager`` allocates through ``gpu_alloc_* / gpu_copy_* /
gpu_dealloc_*`` functions embedded in the payload; here the same three verbs go to the
native library (``lh_b200_malloc / lh_b200_memcpy / lh_b200_free``). The constructor takes
the execution engine, which for this backend is a ``CudaContext``.
"""

from __future__ import annotations

import abc
import ctypes
from contextlib import contextmanager
from dataclasses import dataclass, field

import numpy as np

from ..utils.memref import make_descriptor
from ..utils.numpy import mlir_to_numpy_dtype, numpy_to_mlir_type
from .._native import contiguous_strides


class MemoryManager(abc.ABC):
    """Abstract base class for memory management."""

    @abc.abstractmethod
    def alloc(self, name: str | None = None, **kwargs) -> ctypes.Structure:
        """Allocate a device buffer and return a memref descriptor."""

    @abc.abstractmethod
    def get(self, name: str) -> ctypes.Structure:
        """Look up a previously allocated device buffer by name."""

    @abc.abstractmethod
    def deallocate_all(self):
        """Deallocate all previously allocated device buffers."""

    @staticmethod
    def emit_memory_management_funcs(payload_module, **kwargs):
        """The reference emits gpu.alloc/copy/dealloc helpers into the payload; nothing to
        emit here, the library owns those verbs."""


@dataclass
class ExternalMemoryManager(MemoryManager, abc.ABC):
    """Pass-through manager: converts caller-owned device buffers to memref descriptors."""

    execution_engine: object = None

    @abc.abstractmethod
    def get_memrefs(self, inputs):
        """Convert inputs to memref descriptors."""

    def alloc(self, name: str | None = None, **kwargs) -> ctypes.Structure:
        raise NotImplementedError("Allocation not supported.")

    def get(self, name: str) -> ctypes.Structure:
        raise NotImplementedError("Lookup not supported.")

    def deallocate_all(self):
        raise NotImplementedError("Deallocation not supported.")


@dataclass
class DeviceMemoryManager(MemoryManager, abc.ABC):
    """Abstract base class for handling memory on accelerator devices."""

    execution_engine: object = None

    @abc.abstractmethod
    def copy(self, src, dst):
        """Copy data to/from externally allocated buffers."""

    @abc.abstractmethod
    def clone_host_buffers(self, host_inputs: list[np.ndarray], names: list[str] | None = None):
        """Context manager for creating device buffers from host inputs."""


@dataclass
class CudaMemoryManager(DeviceMemoryManager):
    """Device buffers from ``lh_b200_malloc``; H2D / D2H through ``lh_b200_memcpy``."""

    allocated_buffers: dict = field(default_factory=dict)
    buf_counter: int = 0

    def alloc(self, shape: tuple[int, ...], elem_type, name: str | None = None) -> ctypes.Structure:
        if name is None:
            name = f"buffer_{self.buf_counter}"
            self.buf_counter += 1
        assert name not in self.allocated_buffers, f"Buffer with name '{name}' already exists."
        np_dtype = mlir_to_numpy_dtype(elem_type) if isinstance(elem_type, str) else np.dtype(elem_type)
        nbytes = int(np.prod(shape, dtype=np.int64)) * np_dtype.itemsize
        ptr = self.execution_engine.malloc(nbytes)
        mref = make_descriptor(ptr, shape, contiguous_strides(shape))
        # the descriptor does not carry the element type, so track it alongside
        self.allocated_buffers[name] = (mref, np_dtype, nbytes)
        return mref

    def get(self, name: str) -> ctypes.Structure:
        assert name in self.allocated_buffers, f"No buffer found with name '{name}'."
        return self.allocated_buffers[name][0]

    def deallocate_all(self):
        for mref, _, _ in self.allocated_buffers.values():
            self.execution_engine.free(mref.allocated)
        self.allocated_buffers.clear()
        self.buf_counter = 0

    def _nbytes_of(self, mref) -> int:
        for m, _, nbytes in self.allocated_buffers.values():
            if m is mref:
                return nbytes
        raise ValueError("memref was not allocated by this manager")

    def copy(self, src, dst):
        """Host numpy array <-> device memref. At least one side must be a numpy array."""
        src_np, dst_np = isinstance(src, np.ndarray), isinstance(dst, np.ndarray)
        if not src_np and not dst_np:
            raise ValueError("At least one of src or dst must be a numpy array.")
        if src_np and dst_np:
            np.copyto(dst, src)
            return
        if src_np:
            host = np.ascontiguousarray(src)
            if host.nbytes != self._nbytes_of(dst):
                raise ValueError("size mismatch between host array and device buffer")
            self.execution_engine.memcpy_h2d(dst.allocated, host.ctypes.data, host.nbytes)
            self.execution_engine.sync()  # the host array may be pageable / temporary
        else:
            if not dst.flags["C_CONTIGUOUS"] or not dst.flags["WRITEABLE"]:
                raise ValueError("destination host array must be C-contiguous and writeable")
            if dst.nbytes != self._nbytes_of(src):
                raise ValueError("size mismatch between device buffer and host array")
            self.execution_engine.memcpy_d2h(dst.ctypes.data, src.allocated, dst.nbytes)

    @contextmanager
    def clone_host_buffers(self, host_inputs: list[np.ndarray], names: list[str] | None = None):
        buffers = []
        try:
            for i, host_arr in enumerate(host_inputs):
                name = names[i] if names is not None else None
                buf = self.alloc(host_arr.shape, numpy_to_mlir_type(host_arr.dtype), name=name)
                self.copy(host_arr, buf)
                buffers.append(buf)
            yield buffers
        finally:
            self.deallocate_all()


# The reference's examples name this class; on this backend it is the CUDA manager.
GPUMemoryManager = CudaMemoryManager


class TorchCudaMemoryManager(ExternalMemoryManager):
    """``torch.Tensor(device="cuda")`` arguments passed through without copies — the
    counterpart of ``TorchMemoryManager`` (lighthouse/ingress/torch/compile.py:42-48)."""

    def __init__(self, execution_engine=None):
        self.execution_engine = execution_engine

    @contextmanager
    def get_memrefs(self, inputs):
        memrefs = []
        for t in inputs:
            if not hasattr(t, "data_ptr") or not t.is_cuda:
                raise ValueError("TorchCudaMemoryManager takes CUDA tensors")
            memrefs.append(make_descriptor(t.data_ptr(), tuple(t.shape), tuple(t.stride())))
        yield memrefs
