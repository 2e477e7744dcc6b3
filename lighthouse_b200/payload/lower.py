"""Payload recognition: ``PayloadModule`` function -> ``Plan``.

This is the step that replaces *lowering + JIT* in the reference. The reference classifies
payloads the same way one level up — ``inspect_payload`` walks a function and labels each
layer matmul / batch_matmul / elemwise / reduction (lighthouse/utils/mlir.py:49-210) and
``infer_parameters`` picks a schedule from that (examples/xegpu/kernel_bench.py:95-212) —
and it fuses in the same places: elementwise consumers into the matmul
(lighthouse/schedule/xegpu/mlp_schedule.py:145-166) and
transpose + batch_matmul + scale + softmax + batch_matmul into flash attention
(lighthouse/dialects/transform/transform_ext/ops/replace_with_fused_attention.py:20-219).

Two phases:
  1. ``recognize``: walk the ops in order with every SSA value mapped to a symbolic tensor
     (a strided view of a buffer slot, a constant fill, an uninitialised ``tensor.empty``,
     a row reduction, ...). Views, transposes, broadcasts and reshapes cost nothing; every
     op that computes becomes one plan operator.
  2. ``fuse``: peephole fusion over the plan (GEMM epilogues, norm + cast, attention).
An op or pattern outside the recognised set raises ``ValueError`` — there is no fallback.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from ..plan import ArgSpec, Plan, PlanOp, PView
from .ir import AffineMap, Func, Operation, PayloadModule, ShapedType, Value


class UnsupportedPayload(ValueError):
    pass


@dataclass
class TV:
    """Symbolic tensor value during recognition."""

    kind: str  # view | fill | empty | scalar | rowsum | varsum
    shape: tuple = ()
    dtype: str = "f32"
    view: PView | None = None  # kind == view; for fill: preferred destination (or None)
    scalar: float = 0.0
    src: object = None  # rowsum: TV of x; varsum: (TV of x, inv_n)


# ------------------------------------------------------------------ generic-body expressions
def _expr_of_region(op: Operation, env: dict) -> tuple:
    """Expression tree of the value a linalg.generic yields, over ('arg', i) leaves (block
    argument i = i-th of ins then outs) and ('const', v) leaves (captured constants)."""
    block = op.region
    table: dict[int, tuple] = {id(a): ("arg", i) for i, a in enumerate(block.args)}

    def leaf(v: Value) -> tuple:
        if id(v) in table:
            return table[id(v)]
        tv = env.get(id(v))
        if tv is not None and tv.kind == "scalar":
            return ("const", float(tv.scalar))
        raise UnsupportedPayload(f"linalg.generic body uses {v.name}, which is neither a block argument nor a constant")

    for inner in block.ops:
        if inner.name == "linalg.yield":
            if len(inner.operands) != 1:
                raise UnsupportedPayload("linalg.generic must yield exactly one value")
            return leaf(inner.operands[0])
        if inner.name == "arith.constant":
            table[id(inner.result)] = ("const", float(inner.attrs["value"]))
            continue
        if inner.name == "linalg.index":
            table[id(inner.result)] = ("op", "linalg.index", int(inner.attrs["dim"]))
            continue
        extra = (inner.attrs.get("predicate"),) if inner.name in ("arith.cmpf", "arith.cmpi") else ()
        table[id(inner.result)] = ("op", inner.name) + extra + tuple(leaf(o) for o in inner.operands)
    raise UnsupportedPayload("linalg.generic body has no linalg.yield")


def _is(e, name, n=None) -> bool:
    return isinstance(e, tuple) and e[0] == "op" and e[1] == name and (n is None or len(e) == 2 + n)


def _const(e, value=None) -> bool:
    return isinstance(e, tuple) and e[0] == "const" and (value is None or e[1] == value)


def _arg(e, idx=None) -> bool:
    return isinstance(e, tuple) and e[0] == "arg" and (idx is None or e[1] == idx)


def _commutative_pair(e, pred_a, pred_b):
    """For a binary op expression returns (x, y) with pred_a(x) and pred_b(y), or None."""
    if len(e) != 4:
        return None
    a, b = e[2], e[3]
    if pred_a(a) and pred_b(b):
        return a, b
    if pred_a(b) and pred_b(a):
        return b, a
    return None


from .lower_llama import LlamaPatterns  # noqa: E402  (needs the helpers above)


class Recognizer(LlamaPatterns):
    def __init__(self, func: Func):
        if func.body is None:
            raise UnsupportedPayload(f"function @{func.name} has no body")
        self.func = func
        args = []
        for a in func.args:
            if not isinstance(a.type, ShapedType):
                raise UnsupportedPayload(f"argument {a.name} of @{func.name} is not a tensor or memref")
            if a.type.strides is not None:
                raise UnsupportedPayload("strided function arguments are not supported")
            args.append(ArgSpec(tuple(a.type.shape), a.type.dtype, a.name.lstrip("%")))
        self.plan = Plan(func.name, args)
        self.env: dict[int, TV] = {}
        for i, a in enumerate(func.args):
            self.env[id(a)] = TV("view", a.type.shape, a.type.dtype, self.plan.arg(i))

    # -- helpers --------------------------------------------------------------------------
    def tv(self, v: Value) -> TV:
        if id(v) not in self.env:
            raise UnsupportedPayload(f"value {v.name} has no recognised producer")
        return self.env[id(v)]

    def bind(self, op: Operation, tv: TV) -> None:
        if op.results:
            self.env[id(op.results[0])] = tv

    def as_view(self, tv: TV, what: str) -> PView:
        """A readable buffer view of a symbolic tensor (materialising a constant fill)."""
        if tv.kind == "view":
            return tv.view
        if tv.kind == "fill":
            dst = self.plan.temp(tv.shape, tv.dtype)
            self.plan.elementwise("fill", dst, scalar=tv.scalar)
            return dst
        if tv.kind == "empty":
            raise UnsupportedPayload(f"{what}: reads an uninitialised tensor (tensor.empty)")
        raise UnsupportedPayload(f"{what}: operand is '{tv.kind}', expected a tensor with data")

    def dest_for(self, out_tv: TV, shape=None, dtype=None) -> PView:
        """Where an op writes: the outs operand's buffer when it has one, else a new temporary."""
        if out_tv.kind == "view":
            return out_tv.view
        if out_tv.kind == "fill" and out_tv.view is not None:
            return out_tv.view
        return self.plan.temp(shape or out_tv.shape, dtype or out_tv.dtype)

    # -- main walk ---------------------------------------------------------------------------
    def run(self) -> Plan:
        for op in self.func.body.ops:
            handler = getattr(self, "op_" + op.name.replace(".", "_"), None)
            if handler is None:
                raise UnsupportedPayload(f"Unsupported payload op '{op.name}'")
            handler(op)
        return self.plan

    # -- trivial / view ops ---------------------------------------------------------------------
    def op_arith_constant(self, op):
        self.bind(op, TV("scalar", (), op.result.type, scalar=float(op.attrs["value"])))

    def op_tensor_empty(self, op):
        t = op.result.type
        self.bind(op, TV("empty", t.shape, t.dtype))

    def op_bufferization_to_tensor(self, op):
        self.bind(op, self.tv(op.operands[0]))

    def _alloc(self, op):
        t = op.result.type
        self.bind(op, TV("view", t.shape, t.dtype, self.plan.temp(t.shape, t.dtype)))

    op_gpu_alloc = _alloc
    op_memref_alloc = _alloc

    def _noop(self, op):
        pass

    op_gpu_dealloc = _noop
    op_memref_dealloc = _noop

    def _reshape(self, op):
        src = self.tv(op.operands[0])
        t = op.result.type
        if src.kind != "view":
            self.bind(op, TV(src.kind, t.shape, src.dtype, None, src.scalar, src.src))
            return
        try:
            self.bind(op, TV("view", t.shape, t.dtype, src.view.reshape(t.shape)))
        except ValueError as e:
            raise UnsupportedPayload(f"{op.name}: {e}")

    op_memref_collapse_shape = _reshape
    op_memref_expand_shape = _reshape
    op_tensor_collapse_shape = _reshape
    op_tensor_expand_shape = _reshape

    def op_memref_transpose(self, op):
        src = self.as_view(self.tv(op.operands[0]), "memref.transpose")
        v = src.permute(op.attrs["permutation"])
        self.bind(op, TV("view", v.shape, v.dtype, v))

    def op_linalg_transpose(self, op):
        if self.llama_transpose(op):
            return
        src = self.as_view(self.tv(op.ins[0]), "linalg.transpose")
        v = src.permute(op.attrs["permutation"])
        out = self.tv(op.outs[0])
        if out.kind == "view":  # a transpose into a real buffer is a copy
            self.plan.elementwise("copy", out.view, v)
            self.bind(op, out)
        else:
            self.bind(op, TV("view", v.shape, v.dtype, v))

    def op_linalg_broadcast(self, op):
        out_t = op.outs[0].type
        if self.tv(op.ins[0]).kind == "fill":  # a broadcast constant is still that constant
            return self.bind(op, TV("fill", out_t.shape, out_t.dtype, None, self.tv(op.ins[0]).scalar))
        src = self.as_view(self.tv(op.ins[0]), "linalg.broadcast")
        v = src.broadcast_to(out_t.shape, set(op.attrs["dimensions"]))
        self.bind(op, TV("view", v.shape, v.dtype, v))

    def op_linalg_fill(self, op):
        s = self.tv(op.ins[0])
        if s.kind != "scalar":
            raise UnsupportedPayload("linalg.fill of a non-constant")
        out = self.tv(op.outs[0])
        dest = out.view if out.kind == "view" else None
        if not op.results:  # memref semantics: the fill is a side effect
            if dest is None:
                raise UnsupportedPayload("linalg.fill into a buffer without storage")
            self.plan.elementwise("fill", dest, scalar=s.scalar)
            return
        self.bind(op, TV("fill", op.outs[0].type.shape, op.outs[0].type.dtype, dest, s.scalar))

    def op_linalg_copy(self, op):
        src = self.as_view(self.tv(op.ins[0]), "linalg.copy")
        if self.tv(op.outs[0]).kind == "empty" and op.results:  # copy into a fresh tensor: the source itself will do
            return self.bind(op, TV("view", src.shape, src.dtype, src))
        dst = self.dest_for(self.tv(op.outs[0]))
        self.plan.elementwise("copy", dst, src)
        self.bind(op, TV("view", dst.shape, dst.dtype, dst))

    def op_memref_copy(self, op):
        src = self.as_view(self.tv(op.operands[0]), "memref.copy")
        dst = self.as_view(self.tv(op.operands[1]), "memref.copy")
        self.plan.elementwise("copy", dst, src)

    def op_gpu_memcpy(self, op):
        dst = self.as_view(self.tv(op.operands[0]), "gpu.memcpy")
        src = self.as_view(self.tv(op.operands[1]), "gpu.memcpy")
        self.plan.elementwise("copy", dst, src)

    # -- contractions -----------------------------------------------------------------------------
    def _matmul(self, op, transpose_b=False):
        a = self.as_view(self.tv(op.ins[0]), op.name)
        b = self.as_view(self.tv(op.ins[1]), op.name)
        if transpose_b:
            b = b.t()
        acc = self.tv(op.outs[0])
        out_t = op.outs[0].type
        c = None
        if acc.kind == "view":
            dest = acc.view
            c = acc.view  # accumulate into the existing contents, in place
        elif acc.kind == "fill":
            dest = acc.view if acc.view is not None else self.plan.temp(out_t.shape, out_t.dtype)
            if acc.scalar != 0.0:
                self.plan.elementwise("fill", dest, scalar=acc.scalar)
                c = dest
        elif acc.kind == "empty":
            raise UnsupportedPayload(f"{op.name} accumulates into an uninitialised tensor")
        else:
            raise UnsupportedPayload(f"{op.name}: unsupported accumulator '{acc.kind}'")
        self.plan.gemm(dest, a, b, c=c)
        self.bind(op, TV("view", dest.shape, dest.dtype, dest))

    def op_linalg_matmul(self, op):
        self._matmul(op)

    def op_linalg_batch_matmul(self, op):
        self._matmul(op)

    def op_linalg_matmul_transpose_b(self, op):
        self._matmul(op, transpose_b=True)

    def op_linalg_batch_matmul_transpose_b(self, op):
        self._matmul(op, transpose_b=True)

    # -- named elementwise ops ------------------------------------------------------------------------
    def _binary(self, op, kind):
        x, y = self.tv(op.ins[0]), self.tv(op.ins[1])
        out = self.tv(op.outs[0])
        out_t = op.outs[0].type
        # one operand is a constant fill: scale / relu / identity
        for t, other in ((x, y), (y, x)):
            if other.kind == "fill" and t.kind == "view":
                s = other.scalar
                if kind == "mul":
                    dst = self.dest_for(out, out_t.shape, out_t.dtype)
                    self.plan.elementwise("scale", dst, t.view, scalar=s)
                    return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
                if kind == "max" and s == 0.0:
                    dst = self.dest_for(out, out_t.shape, out_t.dtype)
                    self.plan.elementwise("act", dst, t.view, act="relu")
                    return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
                if kind in ("add", "sub") and s == 0.0 and (kind == "add" or other is y):
                    return self.bind(op, t)
        a = self.as_view(x, op.name)
        b = self.as_view(y, op.name)
        dst = self.dest_for(out, out_t.shape, out_t.dtype)
        self.plan.elementwise(kind, dst, a, b)
        self.bind(op, TV("view", dst.shape, dst.dtype, dst))

    def op_linalg_add(self, op): self._binary(op, "add")
    def op_linalg_sub(self, op): self._binary(op, "sub")
    def op_linalg_mul(self, op): self._binary(op, "mul")
    def op_linalg_max(self, op): self._binary(op, "max")

    def op_linalg_softmax(self, op):
        if self.llama_softmax(op):
            return
        x = self.as_view(self.tv(op.ins[0]), "linalg.softmax")
        if op.attrs.get("dimension") != x.rank - 1:
            raise UnsupportedPayload("linalg.softmax is only supported over the last dimension")
        out_t = op.outs[0].type
        dst = self.dest_for(self.tv(op.outs[0]), out_t.shape, out_t.dtype)
        self.plan.softmax(dst, x)
        self.bind(op, TV("view", dst.shape, dst.dtype, dst))

    # -- linalg.generic ----------------------------------------------------------------------------------
    def op_linalg_generic(self, op):
        maps: list[AffineMap] = op.attrs["indexing_maps"]
        iters = [str(i) for i in op.attrs["iterator_types"]]
        e = _expr_of_region(op, self.env)
        if self.try_llama_generic(op, e, maps, iters):
            return
        n_in = len(op.ins)
        out_val = op.outs[0]
        out_tv = self.tv(out_val)
        out_t = out_val.type
        operands = [self.tv(v) for v in op.operands]

        def operand_view(i: int) -> PView:
            """Operand i as a view broadcast to the iteration space via its indexing map."""
            v = self.as_view(operands[i], "linalg.generic")
            m = maps[i]
            if m.is_identity() and v.rank == m.n_dims:
                return v
            if len(m.results) != v.rank:
                raise UnsupportedPayload("indexing map rank does not match its operand")
            missing = set(range(m.n_dims)) - set(m.results)
            if list(m.results) != sorted(m.results):
                order = sorted(range(len(m.results)), key=lambda k: m.results[k])
                v = v.permute(order)
            return v.broadcast_to(out_t.shape, missing)

        if all(i == "parallel" for i in iters):
            out_map_ok = maps[-1].is_identity()
            if not out_map_ok:
                raise UnsupportedPayload("linalg.generic with a permuted output map")
            # cast
            if (_is(e, "arith.truncf", 1) or _is(e, "arith.extf", 1)) and _arg(e[2], 0):
                dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
                self.plan.elementwise("copy", dst, operand_view(0))
                return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
            # layer-norm normalise step
            if self._try_layernorm(op, e, operands, out_tv, out_t):
                return
            # strip "+ 0" identity wraps and a trailing relu
            act = "none"
            if _is(e, "arith.addf", 2) and _commutative_pair(e, lambda x: not _const(x), lambda x: _const(x, 0.0)):
                e = _commutative_pair(e, lambda x: not _const(x), lambda x: _const(x, 0.0))[0]
            relu_inner = self._relu_of(e)
            if relu_inner is not None:
                act, e = "relu", relu_inner
            if _arg(e):
                src = operand_view(e[1])
                dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
                if act == "none":
                    self.plan.elementwise("copy", dst, src)
                else:
                    self.plan.elementwise("act", dst, src, act=act)
                return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
            for name, kind in (("arith.addf", "add"), ("arith.mulf", "mul"), ("arith.subf", "sub"), ("arith.maximumf", "max")):
                if _is(e, name, 2) and _arg(e[2]) and _arg(e[3]):
                    a, b = operand_view(e[2][1]), operand_view(e[3][1])
                    dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
                    if kind == "add" and act != "none":
                        self.plan.elementwise("add_act", dst, a, b, act=act)
                    elif act == "none":
                        self.plan.elementwise(kind, dst, a, b)
                    else:
                        tmp = self.plan.temp(out_t.shape, out_t.dtype)
                        self.plan.elementwise(kind, tmp, a, b)
                        self.plan.elementwise("act", dst, tmp, act=act)
                    return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
            raise UnsupportedPayload(f"Unsupported elementwise linalg.generic body: {e}")

        # matmul written as a generic: (d0,d2) x (d2,d1) -> (d0,d1), mul + add
        if iters == ["parallel", "parallel", "reduction"] and n_in == 2:
            if [m.results for m in maps] == [(0, 2), (2, 1), (0, 1)] and _is(e, "arith.addf", 2):
                pair = _commutative_pair(e, lambda x: _is(x, "arith.mulf", 2), lambda x: _arg(x, 2))
                if pair and {pair[0][2], pair[0][3]} == {("arg", 0), ("arg", 1)}:
                    fake = Operation("linalg.matmul", op.operands, op.results, n_ins=2)
                    return self._matmul(fake)
        # row reductions of the layer norm
        if iters == ["parallel", "reduction"] and [m.results for m in maps[:1]] == [(0, 1)] and maps[-1].results == (0,):
            acc = out_tv
            if acc.kind != "fill" or acc.scalar != 0.0:
                raise UnsupportedPayload("row reduction must accumulate into a zero fill")
            if n_in == 1 and _is(e, "arith.addf", 2) and {e[2], e[3]} == {("arg", 0), ("arg", 1)}:
                return self.bind(op, TV("rowsum", out_t.shape, out_t.dtype, src=operands[0]))
            if n_in == 2 and operands[1].kind == "rowsum" and operands[1].src is operands[0] and _is(e, "arith.addf", 2):
                pair = _commutative_pair(e, lambda x: _is(x, "arith.mulf", 2), lambda x: _arg(x, 2))
                if pair and pair[0][2] == pair[0][3] and _is(pair[0][2], "arith.subf", 2):
                    centered = pair[0][2]
                    if _arg(centered[2], 0) and _is(centered[3], "arith.mulf", 2):
                        mc = _commutative_pair(centered[3], lambda x: _arg(x, 1), lambda x: _const(x))
                        if mc:
                            return self.bind(op, TV("varsum", out_t.shape, out_t.dtype, src=(operands[0], mc[1][1])))
        raise UnsupportedPayload(f"Unsupported linalg.generic (iterators {iters}, body {e})")

    @staticmethod
    def _relu_of(e):
        """x if e is max(x, 0) or select(x > 0, x, 0), else None."""
        if _is(e, "arith.maximumf", 2) or _is(e, "arith.maxnumf", 2):
            pair = _commutative_pair(e, lambda x: not _const(x), lambda x: _const(x, 0.0))
            return pair[0] if pair else None
        if _is(e, "arith.select", 3):
            c, a, b = e[2], e[3], e[4]
            if isinstance(c, tuple) and c[:2] == ("op", "arith.cmpf") and c[2] in ("ugt", "ogt") and c[3] == a and _const(c[4], 0.0) and _const(b, 0.0):
                return a
        return None

    def _try_layernorm(self, op, e, operands, out_tv, out_t) -> bool:
        """add(mul(mul(sub(x, mul(msum, 1/N)), rsqrt(add(mul(vsum, 1/N), eps))), gamma), beta)"""
        if len(op.ins) != 5 or not _is(e, "arith.addf", 2):
            return False
        x, msum, vsum, gamma, beta = operands[:5]
        if msum.kind != "rowsum" or vsum.kind != "varsum" or msum.src is not x or vsum.src[0] is not x:
            return False
        p1 = _commutative_pair(e, lambda t: _is(t, "arith.mulf", 2), lambda t: _arg(t, 4))
        if not p1:
            return False
        p2 = _commutative_pair(p1[0], lambda t: _is(t, "arith.mulf", 2), lambda t: _arg(t, 3))
        if not p2:
            return False
        p3 = _commutative_pair(p2[0], lambda t: _is(t, "arith.subf", 2), lambda t: _is(t, "math.rsqrt", 1))
        if not p3:
            return False
        centered, rs = p3
        if not (_arg(centered[2], 0) and _is(centered[3], "arith.mulf", 2)):
            return False
        mean = _commutative_pair(centered[3], lambda t: _arg(t, 1), lambda t: _const(t))
        var_eps = rs[2]
        if not mean or not _is(var_eps, "arith.addf", 2):
            return False
        pv = _commutative_pair(var_eps, lambda t: _is(t, "arith.mulf", 2), lambda t: _const(t))
        if not pv:
            return False
        var = _commutative_pair(pv[0], lambda t: _arg(t, 2), lambda t: _const(t))
        if not var:
            return False
        n = x.shape[-1]
        for c in (mean[1][1], var[1][1], vsum.src[1]):
            if abs(c * n - 1.0) > 1e-6:
                raise UnsupportedPayload("layer norm: the 1/N constant does not match the row length")
        eps = pv[1][1]
        dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
        self.plan.layernorm(dst, self.as_view(x, "layernorm"), self.as_view(gamma, "layernorm"), self.as_view(beta, "layernorm"), eps)
        self.bind(op, TV("view", dst.shape, dst.dtype, dst))
        return True

    # -- results -----------------------------------------------------------------------------------------------
    def op_bufferization_materialize_in_destination(self, op):
        src_tv = self.tv(op.operands[0])
        dst = self.as_view(self.tv(op.operands[1]), "materialize_in_destination")
        if src_tv.kind == "fill":
            self.plan.elementwise("fill", dst, scalar=src_tv.scalar)
        else:
            src = self.as_view(src_tv, "materialize_in_destination")
            if src != dst:
                if not self._retarget(src, dst):
                    self.plan.elementwise("copy", dst, src)
        if op.results:
            self.bind(op, TV("view", dst.shape, dst.dtype, dst))

    def _retarget(self, src: PView, dst: PView) -> bool:
        """Makes the producer of temporary ``src`` write straight into ``dst`` when ``src`` is
        a whole temporary written by exactly one operator and not read since."""
        nargs = len(self.plan.args)
        if src.slot < nargs or src.offset != 0 or not src.is_contiguous() or src.shape != dst.shape or src.dtype != dst.dtype:
            return False
        writers = [o for o in self.plan.ops if o.operands[0] is not None and o.operands[0].slot == src.slot]
        readers = [o for o in self.plan.ops if any(v is not None and v.slot == src.slot for v in o.operands[1:])]
        if len(writers) != 1 or writers[0].operands[0] != src:
            return False
        w = writers[0]
        if any(r is not w for r in readers):
            return False
        # a GEMM that accumulates into / adds its own destination keeps doing so in the new place
        w.operands = [dst if (v is not None and v == src) else v for v in w.operands]
        for k, tv in self.env.items():
            if tv.kind == "view" and tv.view == src:
                self.env[k] = TV("view", dst.shape, dst.dtype, dst)
        return True

    def _return(self, op):
        nargs = len(self.plan.args)
        for v in op.operands:
            tv = self.tv(v)
            if tv.kind != "view" or tv.view.slot >= nargs:
                raise UnsupportedPayload("payload functions must leave results in their arguments (no returned temporaries)")

    op_return = _return
    op_func_return = _return


# --------------------------------------------------------------------------------- fusion
def _uses(plan: Plan, slot: int):
    writers = [o for o in plan.ops if o.operands[0] is not None and o.operands[0].slot == slot]
    readers = [o for o in plan.ops if any(v is not None and v.slot == slot for v in o.operands[1:])]
    return writers, readers


def _whole_temp(plan: Plan, v: PView) -> bool:
    return v is not None and v.slot >= len(plan.args) and v.offset == 0 and v.is_contiguous()


def _single_use_link(plan: Plan, producer: PlanOp, consumer: PlanOp, v: PView) -> bool:
    """``v`` is a whole temporary written only by ``producer`` and read only by ``consumer``."""
    if not _whole_temp(plan, v):
        return False
    writers, readers = _uses(plan, v.slot)
    return writers == [producer] and readers == [consumer]


def _is_row_vector_bcast(v: PView, n: int) -> bool:
    return v is not None and v.rank >= 1 and v.shape[-1] == n and v.strides[-1] == 1 and all(s == 0 for s in v.strides[:-1])


def _slots(op: PlanOp):
    return {v.slot for v in op.operands if v is not None}


def _widening_copy_source(plan: Plan, v: PView, reader: PlanOp):
    """If ``v`` is a whole temporary produced only by a float-widening copy (the extf of a
    bias vector) and read only by ``reader``, returns (copy op, its source view)."""
    if not _whole_temp(plan, v):
        return None
    writers, readers = _uses(plan, v.slot)
    if len(writers) != 1 or any(r is not reader for r in readers):
        return None
    w = writers[0]
    if w.kind != "elementwise" or w.attrs["ew"] != "copy" or w.operands[0].shape != w.operands[1].shape:
        return None
    if w.operands[1].dtype not in ("bf16", "f16") or v.dtype != "f32":
        return None
    return w, w.operands[1]


def _fold_inplace_consumer(plan: Plan, i: int, g, d) -> bool:
    """The op right after a GEMM updates the GEMM's result in place (``outs`` used as an input,
    the form of the reference's own exemplar, test/opt/pipeline-check.mlir:21-47: matmul,
    bias add and ReLU as three generics over one tensor): fold it into the GEMM's epilogue.
    Nothing is retargeted, so it does not matter which buffer D is or who reads it later."""
    if i + 1 >= len(plan.ops):
        return False
    nxt = plan.ops[i + 1]
    if nxt.kind != "elementwise" or nxt.operands[0] is None or nxt.operands[0] != d:
        return False
    out, a, b = nxt.operands[:3]
    ew, act = nxt.attrs["ew"], nxt.attrs.get("act", "none")
    has_bias, has_act, has_res = g.operands[4] is not None, g.attrs.get("act", "none") != "none", g.operands[5] is not None
    reads_d = [v for v in (a, b) if v is not None and v == d]
    if len(reads_d) != 1:
        return False
    other = b if a == d else a
    n = d.shape[-1]
    if ew == "act" and (act == "relu" or d.dtype == "f32") and not has_act and not has_res:
        g.attrs["act"] = act
    elif ew in ("add", "add_act") and other is not None and _is_row_vector_bcast(other, n) and not has_bias and not has_act and not has_res and d.rank == 2:
        g.operands[4] = PView(other.slot, (n,), (1,), other.dtype, other.offset)
        if ew == "add_act":
            g.attrs["act"] = act
    elif ew == "add" and other is not None and other.shape == d.shape and other.slot != d.slot and not has_res and other.dtype == d.dtype:
        g.operands[5] = other
    else:
        return False
    del plan.ops[i + 1]
    return True


def fuse_gemm_epilogues(plan: Plan) -> int:
    """Folds bias add, cast, ReLU and residual add that consume a GEMM's output into that
    GEMM (the consumers ``get_tileable_consumers`` finds in the reference). The GEMM moves to
    the consumer's position so that operands produced in between (a widened bias) exist."""
    fused = 0
    changed = True
    while changed:
        changed = False
        for i, g in enumerate(plan.ops):
            if g.kind != "gemm" or g.attrs.get("flags", 0) & ~1:  # SwiGLU / forced-SIMT keep their epilogue
                continue
            d = g.operands[0]
            if _fold_inplace_consumer(plan, i, g, d):
                fused += 1
                changed = True
                break
            if not _whole_temp(plan, d) or (g.operands[3] is not None and g.operands[3] == d):
                continue
            writers, readers = _uses(plan, d.slot)
            if writers != [g] or len(readers) != 1:
                continue
            nxt = readers[0]
            j = plan.ops.index(nxt)
            if j <= i or nxt.kind != "elementwise":
                continue
            # nothing in between may write what the GEMM reads
            g_inputs = {v.slot for v in g.operands[1:] if v is not None}
            if any(o.operands[0] is not None and o.operands[0].slot in g_inputs for o in plan.ops[i + 1 : j]):
                continue
            out, a, b = nxt.operands[:3]
            ew, act = nxt.attrs["ew"], nxt.attrs.get("act", "none")
            has_bias, has_act, has_res = g.operands[4] is not None, g.attrs.get("act", "none") != "none", g.operands[5] is not None
            n = d.shape[-1]
            reads_d = [v for v in (a, b) if v is not None and v == d]
            if len(reads_d) != 1 or out.shape != d.shape:
                continue
            other = b if a == d else a
            drop = None
            ok = False
            if ew == "copy" and not has_res:  # cast (or plain copy): D takes the new type
                ok = True
            elif ew == "act" and (act == "relu" or out.dtype == "f32") and not has_act and not has_res:
                # ReLU commutes with the rounding of a narrow result; any other activation is folded
                # only where the un-fused sequence has no rounding in between (f32 results)
                g.attrs["act"] = act
                ok = True
            elif ew in ("add", "add_act") and _is_row_vector_bcast(other, n) and not has_bias and not has_act and not has_res and d.rank == 2:
                bias = PView(other.slot, (n,), (1,), other.dtype, other.offset)
                src = _widening_copy_source(plan, bias, nxt)
                if src is not None and src[1].is_contiguous():
                    drop, bias = src[0], PView(src[1].slot, (n,), (1,), src[1].dtype, src[1].offset)
                g.operands[4] = bias
                if ew == "add_act":
                    g.attrs["act"] = act
                ok = True
            elif ew == "add" and other is not None and other.shape == d.shape and not has_res and other.dtype == out.dtype:
                g.operands[5] = other
                ok = True
            if not ok:
                continue
            g.operands[0] = out
            plan.ops[j] = g
            del plan.ops[i]
            if drop is not None:
                plan.ops.remove(drop)
            fused += 1
            changed = True
            break
    return fused


def fuse_norm_cast(plan: Plan) -> int:
    """layernorm / rmsnorm followed by a cast of its output: the norm writes the narrow type."""
    fused = 0
    i = 0
    while i + 1 < len(plan.ops):
        a, b = plan.ops[i], plan.ops[i + 1]
        if a.kind in ("layernorm", "rmsnorm") and b.kind == "elementwise" and b.attrs["ew"] == "copy":
            d = a.operands[0]
            if b.operands[1] == d and b.operands[0].shape == d.shape and _single_use_link(plan, a, b, d):
                a.operands[0] = b.operands[0]
                del plan.ops[i + 1]
                fused += 1
                continue
        i += 1
    return fused


def fuse_attention(plan: Plan) -> int:
    """batch_matmul(Q, K^T) -> scale -> softmax -> batch_matmul(P, V) becomes one attention
    operator (what ``replace_with_fused_attention`` does in the reference's schedule)."""
    fused = 0
    i = 0
    while i + 3 < len(plan.ops):
        g1, sc, sm, g2 = plan.ops[i : i + 4]
        ok = g1.kind == "gemm" and sc.kind == "elementwise" and sc.attrs["ew"] == "scale" and sm.kind == "softmax" and g2.kind == "gemm"
        if ok:
            s, q, kt = g1.operands[0], g1.operands[1], g1.operands[2]
            ok = (
                all(g.operands[3] is None and g.operands[4] is None and g.operands[5] is None and g.attrs.get("act", "none") == "none" and not g.attrs.get("flags", 0) for g in (g1, g2))
                and sc.operands[1] == s and sm.operands[1] == sc.operands[0] and g2.operands[1] == sm.operands[0]
                and _single_use_link(plan, g1, sc, s) and _single_use_link(plan, sc, sm, sc.operands[0]) and _single_use_link(plan, sm, g2, sm.operands[0])
                and q.rank in (3, 4) and kt.strides[-2] == 1 and q.strides[-1] == 1 and g2.operands[2].strides[-1] == 1
            )
        if ok:
            k = kt.t()  # back to (batch, S_kv, D)
            o, v = g2.operands[0], g2.operands[2]
            plan.ops[i : i + 4] = [PlanOp("attention", [o, q, k, v], {"scale": sc.attrs["scalar"], "causal": False})]
            fused += 1
        i += 1
    return fused


def compact_temps(plan: Plan) -> None:
    """Drops temporaries no operator touches any more and renumbers the rest."""
    nargs = len(plan.args)
    used = sorted({v.slot for o in plan.ops for v in o.operands if v is not None and v.slot >= nargs})
    remap = {old: nargs + i for i, old in enumerate(used)}
    plan.temp_bytes = [plan.temp_bytes[old - nargs] for old in used]
    for o in plan.ops:
        o.operands = [None if v is None else (PView(remap[v.slot], v.shape, v.strides, v.dtype, v.offset) if v.slot >= nargs else v) for v in o.operands]


def recognize(func: Func, fuse: bool = True, fuse_attention_pattern: bool = True) -> Plan:
    plan = Recognizer(func).run()
    if fuse:
        fuse_gemm_epilogues(plan)
        fuse_norm_cast(plan)
        if fuse_attention_pattern:
            fuse_attention(plan)
    compact_temps(plan)
    return plan


def lower_module(pm: PayloadModule, fuse: bool = True, fuse_attention_pattern: bool = True) -> PayloadModule:
    """Recognises every function with a body and attaches the plans to the module."""
    for name, fn in pm.funcs.items():
        if fn.body is None or name.startswith(("gpu_alloc_", "gpu_dealloc_", "gpu_copy_")):
            continue
        pm.plans[name] = recognize(fn, fuse, fuse_attention_pattern)
    if not pm.plans:
        raise UnsupportedPayload("payload module has no function to run")
    return pm
