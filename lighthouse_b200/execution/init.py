"""Kernel-argument initialisation for ``lh-run`` (same contract as
lighthouse/execution/init.py:12-118 in the reference): ``DIMSxTYPExINIT`` strings,
INIT in {0, 1, rnd, id}; ``rnd`` draws ``np.random.rand`` in [0, 1) from numpy's global
generator, so ``np.random.seed`` upstream fixes the values."""

from __future__ import annotations

from enum import Enum

import numpy as np

from ..utils.numpy import mlir_to_numpy_dtype


class InitType(Enum):
    ZERO = "0"
    ONE = "1"
    RANDOM = "rnd"
    IDENTITY = "id"


class KernelArgument:
    """A host array of shape ``dims`` and type ``element_type`` filled according to ``init_type``."""

    def __init__(self, dims: list[int], element_type, init_type: InitType = InitType.ZERO):
        if dims is None or len(dims) == 0 or not all(isinstance(d, int) and d > 0 for d in dims):
            raise ValueError("Dimensions must be a non-empty list of non-zero integers.")
        self.dims = dims
        self.element_type = element_type
        self.init_type = init_type
        self.arg = self.initialize(dims, init_type, element_type)

    def initialize(self, shape, init_type: InitType, element_type) -> np.ndarray:
        if init_type == InitType.ZERO:
            return np.zeros(shape, dtype=element_type)
        if init_type == InitType.ONE:
            return np.ones(shape, dtype=element_type)
        if init_type == InitType.RANDOM:
            return np.random.rand(*shape).astype(element_type)
        if init_type == InitType.IDENTITY:
            if len(shape) != 2 or shape[0] != shape[1]:
                raise ValueError("Identity initializer only works for square matrices.")
            return np.eye(shape[0], dtype=element_type)
        raise ValueError(f"Unsupported initializer type: {init_type}")


class KernelArgumentParser:
    """``MxNx...xTYPExINIT`` -> ``KernelArgument``; a comma separates arguments."""

    @staticmethod
    def parse(shape_str: str) -> KernelArgument:
        parts = shape_str.split("x")
        if len(parts) < 3:
            raise ValueError(f"Invalid shape string: {shape_str}")
        try:
            element_type = mlir_to_numpy_dtype(parts[-2])
        except ValueError:
            raise ValueError(f"Invalid element type in shape string: {shape_str}")
        try:
            dims = [int(d) for d in parts[:-2]]
        except ValueError:
            raise ValueError(f"Invalid dims in shape string: {shape_str}")
        try:
            init_type = InitType(parts[-1])
        except ValueError:
            raise ValueError(f"Invalid init type in shape string: {shape_str}")
        return KernelArgument(dims, element_type, init_type)

    @staticmethod
    def parse_all(shape_str: str) -> list[KernelArgument]:
        return [KernelArgumentParser.parse(s) for s in shape_str.split(",")]
