"""Execution layer with the reference's names (lighthouse/execution/__init__.py):
``Runner`` is the CUDA runner; there is no CPU engine behind it."""

from .init import InitType, KernelArgument, KernelArgumentParser
from .memory_manager import (
    CudaMemoryManager,
    DeviceMemoryManager,
    ExternalMemoryManager,
    GPUMemoryManager,
    MemoryManager,
    TorchCudaMemoryManager,
)
from .runner import CudaRunner, Runner
from .target import TargetInfo

__all__ = [
    "CudaMemoryManager",
    "CudaRunner",
    "DeviceMemoryManager",
    "ExternalMemoryManager",
    "GPUMemoryManager",
    "InitType",
    "KernelArgument",
    "KernelArgumentParser",
    "MemoryManager",
    "Runner",
    "TargetInfo",
    "TorchCudaMemoryManager",
]
