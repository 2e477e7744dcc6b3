"""Host arrays for ``lh-run`` from ``--input-shape`` strings.

Contract of lighthouse/execution/init.py:12-118 in the reference: an argument is written
``DIMSxTYPExINIT`` (``16x64xf32xrnd``), arguments are separated by commas, INIT is one of
``0``, ``1``, ``rnd``, ``id``; ``rnd`` draws ``np.random.rand`` in [0, 1) from numpy's global
generator, so a ``np.random.seed`` upstream fixes the values (the golden vector of the
reference's ``lh-run`` test depends on exactly that draw order).
"""

from __future__ import annotations

import re
from enum import Enum

import numpy as np

from ..utils.numpy import mlir_to_numpy_dtype


class InitType(Enum):
    ZERO = "0"
    ONE = "1"
    RANDOM = "rnd"
    IDENTITY = "id"


def _identity(shape, dtype) -> np.ndarray:
    if len(shape) != 2 or shape[0] != shape[1]:
        raise ValueError("Identity initializer only works for square matrices.")
    return np.eye(shape[0], dtype=dtype)


# one filler per initialiser; each takes (shape, numpy dtype)
_FILLERS = {
    InitType.ZERO: lambda shape, dtype: np.zeros(shape, dtype=dtype),
    InitType.ONE: lambda shape, dtype: np.ones(shape, dtype=dtype),
    InitType.RANDOM: lambda shape, dtype: np.random.rand(*shape).astype(dtype),
    InitType.IDENTITY: _identity,
}


class KernelArgument:
    """``arg`` is the filled host array; ``dims``, ``element_type`` and ``init_type`` are kept
    for whoever prints or re-creates it."""

    def __init__(self, dims: list[int], element_type, init_type: InitType = InitType.ZERO):
        valid = dims is not None and len(dims) > 0 and all(isinstance(d, int) and d > 0 for d in dims)
        if not valid:
            raise ValueError("Dimensions must be a non-empty list of non-zero integers.")
        self.dims, self.element_type, self.init_type = dims, element_type, init_type
        self.arg = self.initialize(dims, init_type, element_type)

    def initialize(self, shape, init_type: InitType, element_type) -> np.ndarray:
        filler = _FILLERS.get(init_type)
        if filler is None:
            raise ValueError(f"Unsupported initializer type: {init_type}")
        return filler(shape, element_type)


_FIELDS = re.compile(r"^(?P<dims>.*)x(?P<type>[^x]*)x(?P<init>[^x]*)$")


class KernelArgumentParser:
    """``MxNx...xTYPExINIT`` -> ``KernelArgument``."""

    @staticmethod
    def parse(shape_str: str) -> KernelArgument:
        m = _FIELDS.match(shape_str)
        if m is None:
            raise ValueError(f"Invalid shape string: {shape_str}")
        try:
            element_type = mlir_to_numpy_dtype(m["type"])
        except ValueError:
            raise ValueError(f"Invalid element type in shape string: {shape_str}") from None
        if not re.fullmatch(r"-?\d+(x-?\d+)*", m["dims"]):
            raise ValueError(f"Invalid dims in shape string: {shape_str}")
        if m["init"] not in {t.value for t in InitType}:
            raise ValueError(f"Invalid init type in shape string: {shape_str}")
        return KernelArgument([int(d) for d in m["dims"].split("x")], element_type, InitType(m["init"]))

    @staticmethod
    def parse_all(shape_str: str) -> list[KernelArgument]:
        return [KernelArgumentParser.parse(field) for field in shape_str.split(",")]
