"""Builder for payload functions: the op-emitting calls the reference's generators make on
the MLIR Python bindings (``linalg.matmul(...)``, ``tensor.empty(...)``,
``bufferization.materialize_in_destination(...)``, ``@linalg.generic`` bodies, ...),
re-created on the in-memory IR of ``ir.py``. Element types are given by name ("f32",
"bf16", "f16")."""

from __future__ import annotations

from .ir import AffineMap, Block, Func, Operation, PayloadModule, ShapedType, Value, memref_t, tensor_t

PARALLEL = "parallel"
REDUCTION = "reduction"


def affine_map(n_dims: int, results) -> AffineMap:
    return AffineMap(n_dims, tuple(results))


def identity_map(rank: int) -> AffineMap:
    return AffineMap(rank, tuple(range(rank)))


class RegionBuilder:
    """Emits scalar ops into a ``linalg.generic`` body."""

    def __init__(self, fb: "FuncBuilder", block: Block):
        self.fb, self.block = fb, block

    def _emit(self, name, operands, type_, **attrs) -> Value:
        op = Operation(name, list(operands), attrs=attrs)
        v = Value(self.fb._fresh(), type_, op)
        op.results.append(v)
        self.block.ops.append(op)
        return v

    def addf(self, a, b): return self._emit("arith.addf", [a, b], a.type)
    def subf(self, a, b): return self._emit("arith.subf", [a, b], a.type)
    def mulf(self, a, b): return self._emit("arith.mulf", [a, b], a.type)
    def divf(self, a, b): return self._emit("arith.divf", [a, b], a.type)
    def maximumf(self, a, b): return self._emit("arith.maximumf", [a, b], a.type)
    def rsqrt(self, a): return self._emit("math.rsqrt", [a], a.type)
    def exp(self, a): return self._emit("math.exp", [a], a.type)
    def truncf(self, a, dtype): return self._emit("arith.truncf", [a], dtype)
    def extf(self, a, dtype): return self._emit("arith.extf", [a], dtype)

    def negf(self, a): return self._emit("arith.negf", [a], a.type)
    def cos(self, a): return self._emit("math.cos", [a], a.type)
    def sin(self, a): return self._emit("math.sin", [a], a.type)
    def complex_create(self, re, im): return self._emit("complex.create", [re, im], f"complex<{re.type}>")
    def complex_mul(self, a, b): return self._emit("complex.mul", [a, b], a.type)
    def complex_re(self, a): return self._emit("complex.re", [a], a.type[len("complex<") : -1])
    def complex_im(self, a): return self._emit("complex.im", [a], a.type[len("complex<") : -1])
    def index(self, dim: int): return self._emit("linalg.index", [], "index", dim=int(dim))
    def cmpi(self, pred, a, b): return self._emit("arith.cmpi", [a, b], "i1", predicate=pred)

    def cmpf(self, pred, a, b): return self._emit("arith.cmpf", [a, b], "i1", predicate=pred)
    def select(self, c, a, b): return self._emit("arith.select", [c, a, b], a.type)


class FuncBuilder:
    def __init__(self, module: PayloadModule, name: str, arg_types: list, arg_names: list[str] | None = None, c_interface: bool = True):
        self.module = module
        self._n = 0
        args = []
        for i, t in enumerate(arg_types):
            nm = f"%{arg_names[i]}" if arg_names else f"%arg{i}"
            args.append(Value(nm, t))
        self.func = Func(name, args, Block(args=list(args)), [], {"llvm.emit_c_interface": True} if c_interface else {})
        module.add(self.func)

    @property
    def args(self) -> list[Value]:
        return self.func.args

    def _fresh(self) -> str:
        name = f"%{self._n}"
        self._n += 1
        return name

    def _emit(self, name, operands, result_types=(), n_ins=0, region=None, **attrs) -> Operation:
        op = Operation(name, list(operands), attrs=dict(attrs), region=region, n_ins=n_ins)
        for t in result_types:
            op.results.append(Value(self._fresh(), t, op))
        self.func.body.ops.append(op)
        return op

    # -- scalars / tensors ---------------------------------------------------------------
    def constant(self, value, dtype: str) -> Value:
        return self._emit("arith.constant", [], [dtype], value=value).result

    def empty(self, shape, dtype: str) -> Value:
        return self._emit("tensor.empty", [], [tensor_t(shape, dtype)]).result

    def to_tensor(self, memref: Value, restrict: bool = True, writable: bool = False) -> Value:
        attrs = {"restrict": True} if restrict else {}
        if writable:
            attrs["writable"] = True
        return self._emit("bufferization.to_tensor", [memref], [memref.type.with_kind("tensor")], **attrs).result

    def materialize_in_destination(self, tensor: Value, memref: Value) -> None:
        self._emit("bufferization.materialize_in_destination", [tensor, memref], [], restrict=True, writable=True)

    # -- linalg named ops -------------------------------------------------------------------
    def _structured(self, name, ins, outs, **attrs) -> Value | None:
        is_tensor = isinstance(outs[0].type, ShapedType) and outs[0].type.kind == "tensor"
        op = self._emit(name, list(ins) + list(outs), [outs[0].type] if is_tensor else [], n_ins=len(ins), **attrs)
        return op.result if is_tensor else None

    def fill(self, scalar: Value, out: Value): return self._structured("linalg.fill", [scalar], [out])
    def matmul(self, a, b, acc): return self._structured("linalg.matmul", [a, b], [acc])
    def batch_matmul(self, a, b, acc): return self._structured("linalg.batch_matmul", [a, b], [acc])
    def add(self, a, b, out): return self._structured("linalg.add", [a, b], [out])
    def sub(self, a, b, out): return self._structured("linalg.sub", [a, b], [out])
    def mul(self, a, b, out): return self._structured("linalg.mul", [a, b], [out])
    def max(self, a, b, out): return self._structured("linalg.max", [a, b], [out])
    def transpose(self, x, out, permutation): return self._structured("linalg.transpose", [x], [out], permutation=list(permutation))
    def broadcast(self, x, out, dimensions): return self._structured("linalg.broadcast", [x], [out], dimensions=list(dimensions))
    def softmax(self, x, out, dimension: int): return self._structured("linalg.softmax", [x], [out], dimension=int(dimension))
    def copy(self, x, out): return self._structured("linalg.copy", [x], [out])

    def contract(self, a, b, out, maps):
        """``linalg.contract``: multiply-accumulate over the dims that appear in ``a``'s and
        ``b``'s maps but not in ``out``'s."""
        return self._structured("linalg.contract", [a, b], [out], indexing_maps=list(maps))

    def elementwise(self, kind: str, ins, out):
        """``linalg.elementwise kind=#linalg.elementwise_kind<kind>`` (add, mul, square, rsqrt, ...)."""
        return self._structured("linalg.elementwise", list(ins), [out], kind=kind)

    def generic(self, ins, outs, maps, iterator_types, body) -> Value | None:
        """``body(rb, *block_args)`` returns the value to yield; block args are the element
        values of ins then outs, as in the bindings' ``@linalg.generic`` decorator."""
        block = Block()
        for v in list(ins) + list(outs):
            t = v.type.dtype if isinstance(v.type, ShapedType) else v.type
            block.args.append(Value(self._fresh().replace("%", "%in"), t))
        rb = RegionBuilder(self, block)
        yielded = body(rb, *block.args)
        block.ops.append(Operation("linalg.yield", [yielded]))
        is_tensor = outs[0].type.kind == "tensor"
        op = self._emit("linalg.generic", list(ins) + list(outs), [outs[0].type] if is_tensor else [], n_ins=len(ins), region=block, indexing_maps=list(maps), iterator_types=list(iterator_types))
        return op.result if is_tensor else None

    # -- memref views / allocation ---------------------------------------------------------
    def collapse_shape(self, m: Value, result_shape, reassociation) -> Value:
        t = ShapedType(m.type.kind, tuple(result_shape), m.type.dtype)
        return self._emit("memref.collapse_shape" if m.type.kind == "memref" else "tensor.collapse_shape", [m], [t], reassociation=[list(g) for g in reassociation]).result

    def expand_shape(self, m: Value, result_shape, reassociation) -> Value:
        t = ShapedType(m.type.kind, tuple(result_shape), m.type.dtype)
        return self._emit("memref.expand_shape" if m.type.kind == "memref" else "tensor.expand_shape", [m], [t], reassociation=[list(g) for g in reassociation], output_shape=list(result_shape)).result

    def memref_transpose(self, m: Value, permutation) -> Value:
        src = m.type
        strides = src.element_strides()
        shape = tuple(src.shape[p] for p in permutation)
        t = memref_t(shape, src.dtype, tuple(strides[p] for p in permutation), src.offset)
        return self._emit("memref.transpose", [m], [t], permutation=list(permutation)).result

    def gpu_alloc(self, shape, dtype: str) -> Value:
        return self._emit("gpu.alloc", [], [memref_t(shape, dtype)]).result

    def gpu_dealloc(self, m: Value) -> None:
        self._emit("gpu.dealloc", [m], [])

    def ret(self, *values) -> None:
        self._emit("return", list(values), [])
        self.func.result_types = [v.type for v in values]
