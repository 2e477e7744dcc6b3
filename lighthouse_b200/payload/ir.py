"""A small in-memory form of the MLIR payload subset this backend recognises.

The reference hands ``ir.Module`` objects of the upstream MLIR Python bindings between its
layers (lighthouse/pipeline/driver.py:155-235, lighthouse/execution/runner.py:49-72).
Those bindings are a third-party package that cannot be assumed here, so payloads are held
in these plain classes instead: enough structure for the ops the payload generators emit
(func, arith, tensor.empty, linalg named ops and generics, bufferization to_tensor /
materialize_in_destination, memref reshapes and transposes, gpu alloc/dealloc), printable
as MLIR text and parsable back from it (``payload/parser.py``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

FLOAT_TYPES = ("f16", "bf16", "f32", "f64")
INT_TYPES = ("i1", "i8", "i16", "i32", "i64", "index")


@dataclass(frozen=True)
class ShapedType:
    """``tensor<...>`` or ``memref<...>`` with a static shape; memrefs may carry a
    ``strided<[...], offset: N>`` layout (strides in elements)."""

    kind: str  # "tensor" | "memref"
    shape: tuple[int, ...]
    dtype: str
    strides: tuple[int, ...] | None = None
    offset: int = 0

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        return math.prod(self.shape)

    def element_strides(self) -> tuple[int, ...]:
        if self.strides is not None:
            return self.strides
        out, acc = [], 1
        for d in reversed(self.shape):
            out.append(acc)
            acc *= d
        return tuple(reversed(out))

    def with_kind(self, kind: str) -> "ShapedType":
        return ShapedType(kind, self.shape, self.dtype, self.strides if kind == "memref" else None, self.offset if kind == "memref" else 0)

    def __str__(self) -> str:
        dims = "x".join(str(d) for d in self.shape)
        body = f"{dims}x{self.dtype}" if self.shape else self.dtype
        if self.kind == "memref" and self.strides is not None:
            layout = f"strided<[{', '.join(str(s) for s in self.strides)}]"
            if self.offset:
                layout += f", offset: {self.offset}"
            body += f", {layout}>"
        return f"{self.kind}<{body}>"


def tensor_t(shape, dtype: str) -> ShapedType:
    return ShapedType("tensor", tuple(int(d) for d in shape), dtype)


def memref_t(shape, dtype: str, strides=None, offset: int = 0) -> ShapedType:
    return ShapedType("memref", tuple(int(d) for d in shape), dtype, None if strides is None else tuple(int(s) for s in strides), offset)


@dataclass(eq=False)
class Value:
    name: str  # with the leading '%'
    type: object  # ShapedType | str (scalar type name)
    owner: "Operation | None" = None  # defining op (None for block/function arguments)

    def __str__(self) -> str:
        return self.name


@dataclass(eq=False)
class Block:
    args: list[Value] = field(default_factory=list)
    ops: list["Operation"] = field(default_factory=list)


@dataclass(eq=False)
class Operation:
    name: str  # e.g. "linalg.matmul"
    operands: list[Value] = field(default_factory=list)
    results: list[Value] = field(default_factory=list)
    attrs: dict = field(default_factory=dict)
    region: Block | None = None
    # linalg structured ops keep the ins / outs split
    n_ins: int = 0

    @property
    def ins(self) -> list[Value]:
        return self.operands[: self.n_ins]

    @property
    def outs(self) -> list[Value]:
        return self.operands[self.n_ins :]

    @property
    def result(self) -> Value:
        return self.results[0]


@dataclass(eq=False)
class AffineMap:
    """``affine_map<(d0, d1, ...) -> (exprs)>`` with results that are single dims (projected
    permutations, which is all the GPU payload generics use) and, for the Llama builders,
    constants (``(d0, d1) -> (d0, 0)``) and floor divisions of a dim by a constant
    (``d2 floordiv 4``). ``results[i]`` is the dim index of result i (-1 for a constant);
    ``special`` holds, per result index, ``("const", value)`` or ``("floordiv", divisor)``."""

    n_dims: int
    results: tuple[int, ...]  # dim index per result
    special: dict = field(default_factory=dict)

    def _expr(self, i: int) -> str:
        sp = self.special.get(i)
        if sp is None:
            return f"d{self.results[i]}"
        if sp[0] == "const":
            return str(sp[1])
        return f"d{self.results[i]} floordiv {sp[1]}"

    def __str__(self) -> str:
        dims = ", ".join(f"d{i}" for i in range(self.n_dims))
        res = ", ".join(self._expr(i) for i in range(len(self.results)))
        return f"affine_map<({dims}) -> ({res})>"

    def is_plain(self) -> bool:
        return not self.special

    def is_identity(self) -> bool:
        return not self.special and self.results == tuple(range(self.n_dims))


@dataclass(eq=False)
class Func:
    name: str
    args: list[Value]
    body: Block | None  # None for declarations
    result_types: list = field(default_factory=list)
    attrs: dict = field(default_factory=dict)


class PayloadModule:
    """A parsed (or built) payload: functions by name, plus what the CUDA dispatch stage
    attaches — ``plans`` (function name -> ``Plan``) and ``bench_target``."""

    def __init__(self):
        self.funcs: dict[str, Func] = {}
        self.plans: dict = {}
        self.bench_target: str | None = None
        self.source_path: str | None = None

    def add(self, func: Func) -> Func:
        if func.name in self.funcs:
            raise ValueError(f"redefinition of function @{func.name}")
        self.funcs[func.name] = func
        return func

    def __str__(self) -> str:
        from .printer import print_module

        return print_module(self)
