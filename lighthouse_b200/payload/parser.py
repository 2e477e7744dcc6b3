"""Reader for the textual form of the MLIR payload subset (see ``ir.py``).

It accepts what ``str(ir.Module)`` prints for the ops the reference's payload generators
emit — the custom assembly of func / arith / math / tensor / linalg / bufferization /
memref / gpu ops — and raises ``ValueError`` on anything else, which is how an unsupported
payload is reported (the reference's dispatcher does the same,
examples/xegpu/kernel_bench.py:95-212). Textual exemplars in the reference:
test/run/pipeline-check.mlir:7-14, test/opt/pipeline-check.mlir:21-47,
test/transform/test_tile_and_fuse.py:58-131,505-529.
"""

from __future__ import annotations

import re

from .ir import AffineMap, Block, Func, Operation, PayloadModule, ShapedType, Value

_WS = re.compile(r"(?:\s+|//[^\n]*)*")
_SSA = re.compile(r"%[A-Za-z0-9_$.\-]+(?:#\d+)?")
_IDENT = re.compile(r"[A-Za-z_][A-Za-z0-9_$.]*")
_NUMBER = re.compile(r"[-+]?(?:0x[0-9a-fA-F]+|(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?|inf|nan)")
_SCALAR_TYPE = re.compile(r"(?:complex<(?:bf16|f16|f32|f64)>|(?:bf16|f16|f32|f64|index|i\d+)\b)")

ELEMENTWISE_BINARY = {"add", "sub", "mul", "div", "max", "min"}
ELEMENTWISE_UNARY = {"exp", "log", "abs", "negf", "tanh", "erf", "sqrt", "rsqrt", "floor", "ceil", "square", "reciprocal"}
REGION_BINARY = {
    "arith.addf", "arith.subf", "arith.mulf", "arith.divf", "arith.maximumf", "arith.maxnumf", "arith.minimumf", "arith.minnumf",
    "arith.addi", "arith.muli", "arith.subi", "complex.mul",
}
REGION_UNARY = {"arith.negf", "math.rsqrt", "math.sqrt", "math.exp", "math.tanh", "math.erf", "math.log", "math.absf", "math.exp2", "math.cos", "math.sin"}
REGION_CAST = {"arith.truncf", "arith.extf", "arith.sitofp", "arith.uitofp", "arith.fptosi", "arith.index_cast", "arith.bitcast"}


class ParseError(ValueError):
    pass


class _Parser:
    def __init__(self, text: str):
        self.t = text
        self.i = 0
        self.maps: dict[str, AffineMap] = {}
        self.scopes: list[dict[str, Value]] = []

    # ---------------------------------------------------------------- scanning helpers
    def ws(self) -> None:
        self.i = _WS.match(self.t, self.i).end()

    def eof(self) -> bool:
        self.ws()
        return self.i >= len(self.t)

    def fail(self, msg: str):
        line = self.t.count("\n", 0, self.i) + 1
        snippet = self.t[self.i : self.i + 60].split("\n")[0]
        raise ParseError(f"MLIR payload line {line}: {msg} (at '{snippet}')")

    def peek(self, lit: str) -> bool:
        self.ws()
        return self.t.startswith(lit, self.i)

    def accept(self, lit: str) -> bool:
        if self.peek(lit):
            self.i += len(lit)
            return True
        return False

    def accept_word(self, word: str) -> bool:
        self.ws()
        if self.t.startswith(word, self.i):
            end = self.i + len(word)
            if end >= len(self.t) or not (self.t[end].isalnum() or self.t[end] in "_."):
                self.i = end
                return True
        return False

    def expect(self, lit: str) -> None:
        if not self.accept(lit):
            self.fail(f"expected '{lit}'")

    def rx(self, pat: re.Pattern):
        self.ws()
        m = pat.match(self.t, self.i)
        if m:
            self.i = m.end()
        return m

    def ident(self) -> str:
        m = self.rx(_IDENT)
        if not m:
            self.fail("expected identifier")
        return m.group(0)

    def integer(self) -> int:
        m = self.rx(re.compile(r"-?\d+"))
        if not m:
            self.fail("expected integer")
        return int(m.group(0))

    def int_list(self) -> list[int]:
        self.expect("[")
        out = []
        if not self.accept("]"):
            while True:
                out.append(self.integer())
                if self.accept("]"):
                    break
                self.expect(",")
        return out

    def balanced(self, open_ch: str, close_ch: str) -> str:
        """Consumes a balanced bracket group starting at the cursor and returns its inside."""
        self.ws()
        if not self.t.startswith(open_ch, self.i):
            self.fail(f"expected '{open_ch}'")
        depth, j = 0, self.i
        in_str = False
        while j < len(self.t):
            c = self.t[j]
            if in_str:
                if c == '"':
                    in_str = False
            elif c == '"':
                in_str = True
            elif c == open_ch:
                depth += 1
            elif c == close_ch:
                if not (close_ch == ">" and j > 0 and self.t[j - 1] == "-"):  # '->' inside affine_map
                    depth -= 1
                    if depth == 0:
                        inner = self.t[self.i + 1 : j]
                        self.i = j + 1
                        return inner
            j += 1
        self.fail(f"unbalanced '{open_ch}'")

    # ------------------------------------------------------------------------- types
    def type(self):
        self.ws()
        for kind in ("tensor", "memref"):
            if self.t.startswith(kind + "<", self.i):
                self.i += len(kind)
                return self._shaped(kind, self.balanced("<", ">"))
        m = self.rx(_SCALAR_TYPE)
        if m:
            return m.group(0)
        if self.accept("("):  # function type "() -> ()" or tuple of types; only "()" needed
            self.expect(")")
            return "()"
        self.fail("expected a type")

    def _shaped(self, kind: str, inner: str) -> ShapedType:
        head, _, layout = inner.partition(",")
        head = head.strip()
        tail = re.search(r"(complex<\w+>|bf16|f16|f32|f64|index|i\d+)$", head)  # the element type may itself contain an 'x'
        dtype = tail.group(1) if tail else ""
        if not _SCALAR_TYPE.fullmatch(dtype):
            raise ParseError(f"unsupported element type in {kind}<{inner}>")
        dims = []
        for d in [x for x in head[: tail.start()].split("x") if x.strip()]:
            d = d.strip()
            if d == "?":
                raise ParseError(f"dynamic shapes are not supported: {kind}<{inner}>")
            dims.append(int(d))
        strides, offset = None, 0
        layout = layout.strip()
        if layout:
            m = re.match(r"strided<\[([^\]]*)\](?:\s*,\s*offset:\s*(-?\d+|\?))?>", layout)
            if not m:
                raise ParseError(f"unsupported memref layout '{layout}'")
            strides = tuple(int(s) for s in m.group(1).split(",") if s.strip())
            if m.group(2) == "?":
                raise ParseError("dynamic memref offsets are not supported")
            offset = int(m.group(2)) if m.group(2) else 0
        return ShapedType(kind, tuple(dims), dtype, strides, offset)

    def affine_map(self) -> AffineMap:
        self.ws()
        if self.peek("#"):
            self.i += 1
            name = self.ident()
            if name not in self.maps:
                self.fail(f"unknown affine map alias #{name}")
            return self.maps[name]
        if not self.accept_word("affine_map"):
            self.fail("expected affine_map")
        return self._affine_map_body(self.balanced("<", ">"))

    @staticmethod
    def _affine_map_body(inner: str) -> AffineMap:
        m = re.fullmatch(r"\s*\(([^)]*)\)\s*(?:\[[^\]]*\]\s*)?->\s*\(([^)]*)\)\s*", inner)
        if not m:
            raise ParseError(f"unsupported affine_map<{inner}>")
        dims = [d.strip() for d in m.group(1).split(",") if d.strip()]
        results, special = [], {}
        for r in (x.strip() for x in m.group(2).split(",")):
            if not r:
                continue
            fd = re.fullmatch(r"(\w+)\s+floordiv\s+(\d+)", r)
            if r in dims:
                results.append(dims.index(r))
            elif re.fullmatch(r"-?\d+", r):
                special[len(results)] = ("const", int(r))
                results.append(-1)
            elif fd and fd.group(1) in dims:
                special[len(results)] = ("floordiv", int(fd.group(2)))
                results.append(dims.index(fd.group(1)))
            else:
                raise ParseError(f"affine_map result '{r}' is not a dimension, a constant or 'dim floordiv constant'")
        return AffineMap(len(dims), tuple(results), special)

    # ------------------------------------------------------------------------- values
    def define(self, name: str, type_, owner=None) -> Value:
        v = Value(name, type_, owner)
        self.scopes[-1][name] = v
        return v

    def use(self, name: str) -> Value:
        for scope in reversed(self.scopes):
            if name in scope:
                return scope[name]
        self.fail(f"use of undefined value {name}")

    def ssa_use(self) -> Value:
        m = self.rx(_SSA)
        if not m:
            self.fail("expected an SSA value")
        return self.use(m.group(0))

    def attr_value(self):
        self.ws()
        if self.peek("["):
            self.expect("[")
            out = []
            if not self.accept("]"):
                while True:
                    out.append(self.attr_value())
                    if self.accept("]"):
                        break
                    self.expect(",")
            return out
        if self.peek('"'):
            m = self.rx(re.compile(r'"((?:[^"\\]|\\.)*)"'))
            return m.group(1)
        if self.peek("#") and not self.t.startswith("#linalg", self.i):
            return self.affine_map()
        if self.t.startswith("affine_map", self.i):
            return self.affine_map()
        if self.peek("#"):  # dialect attribute such as #linalg.iterator_type<parallel>
            m = self.rx(re.compile(r"#[A-Za-z_.]+(?:<[^>]*>)?"))
            inner = re.search(r"<([^>]*)>", m.group(0))
            return inner.group(1) if inner else m.group(0)
        if self.accept_word("true"):
            return True
        if self.accept_word("false"):
            return False
        if self.accept_word("unit"):
            return True
        if self.accept_word("dense"):
            return ("dense", self.balanced("<", ">"))
        m = self.rx(_NUMBER)
        if m:
            txt = m.group(0)
            val = float(txt) if any(c in txt for c in ".eEn") and not txt.startswith("0x") else int(txt, 0)
            if self.accept(":"):
                self.type()
            return val
        m = self.rx(_IDENT)
        if m:
            return m.group(0)
        self.fail("unsupported attribute value")

    def attr_dict(self) -> dict:
        self.expect("{")
        out = {}
        if self.accept("}"):
            return out
        while True:
            self.ws()
            m = self.rx(re.compile(r'"[^"]+"|[A-Za-z_][A-Za-z0-9_.$]*'))
            if not m:
                self.fail("expected attribute name")
            key = m.group(0).strip('"')
            out[key] = self.attr_value() if self.accept("=") else True
            if self.accept("}"):
                return out
            self.expect(",")

    # ---------------------------------------------------------------------- top level
    def module(self) -> PayloadModule:
        pm = PayloadModule()
        self.scopes.append({})
        wrapped = False
        while not self.eof():
            if self.peek("#"):
                self.i += 1
                name = self.ident()
                self.expect("=")
                if self.accept_word("affine_map"):
                    self.maps[name] = self._affine_map_body(self.balanced("<", ">"))
                else:  # some other attribute alias: skip to end of line
                    nl = self.t.find("\n", self.i)
                    self.i = len(self.t) if nl < 0 else nl
            elif self.accept_word("module") or self.accept_word("builtin.module"):
                if self.peek("@"):
                    self.i += 1
                    self.ident()
                if self.accept_word("attributes"):
                    self.attr_dict()
                self.expect("{")
                wrapped = True
            elif self.peek("}"):
                if not wrapped:
                    self.fail("unexpected '}'")
                self.i += 1
                wrapped = False
            elif self.accept_word("func.func"):
                self.func(pm)
            else:
                self.fail("expected 'module' or 'func.func'")
        return pm

    def func(self, pm: PayloadModule) -> None:
        attrs = {}
        for vis in ("private", "public", "nested"):
            if self.accept_word(vis):
                attrs["visibility"] = vis
        self.expect("@")
        name = self.ident()
        self.scopes.append({})
        self.expect("(")
        args, decl_types = [], []
        if not self.accept(")"):
            while True:
                m = self.rx(_SSA)
                if m:
                    self.expect(":")
                    t = self.type()
                    if self.peek("{"):
                        self.attr_dict()
                    args.append(self.define(m.group(0), t))
                else:
                    decl_types.append(self.type())
                if self.accept(")"):
                    break
                self.expect(",")
        results = []
        if self.accept("->"):
            if self.accept("("):
                if not self.accept(")"):
                    while True:
                        results.append(self.type())
                        if self.accept(")"):
                            break
                        self.expect(",")
            else:
                results.append(self.type())
        if self.accept_word("attributes"):
            attrs.update(self.attr_dict())
        body = None
        if self.peek("{"):
            self.expect("{")
            body = Block(args=args)
            while not self.accept("}"):
                body.ops.append(self.operation())
        self.scopes.pop()
        pm.add(Func(name, args, body, results, attrs))

    # --------------------------------------------------------------------- operations
    def operation(self) -> Operation:
        self.ws()
        result_names = []
        if self.peek("%"):
            while True:
                m = self.rx(re.compile(r"%[A-Za-z0-9_$.\-]+(?::\d+)?"))
                result_names.append(m.group(0).split(":")[0])
                if not self.accept(","):
                    break
            self.expect("=")
        name = self.ident()
        op = Operation(name)
        handler = getattr(self, "_op_" + name.replace(".", "_"), None)
        if handler is not None:
            types = handler(op)
        elif name.startswith("linalg.") and name.split(".", 1)[1] in (
            ELEMENTWISE_BINARY | ELEMENTWISE_UNARY | {"matmul", "batch_matmul", "fill", "transpose", "broadcast", "softmax", "generic", "copy", "matmul_transpose_b", "matmul_transpose_a", "batch_matmul_transpose_b", "contract", "elementwise"}
        ):
            types = self._linalg_structured(op)
        elif name in REGION_BINARY:
            a = self.ssa_use()
            self.expect(",")
            b = self.ssa_use()
            self._fastmath()
            self.expect(":")
            t = self.type()
            op.operands, types = [a, b], [t]
        elif name in REGION_UNARY:
            a = self.ssa_use()
            self._fastmath()
            self.expect(":")
            t = self.type()
            op.operands, types = [a], [t]
        elif name in REGION_CAST:
            a = self.ssa_use()
            self._fastmath()
            self.expect(":")
            self.type()
            if not self.accept_word("to"):
                self.fail("expected 'to' in cast")
            t = self.type()
            op.operands, types = [a], [t]
        else:
            self.fail(f"Unsupported op '{name}' in payload")
        if len(types) != len(result_names):
            if result_names and not types:
                self.fail(f"op '{name}' defines results but none were parsed")
            if len(result_names) == 0:
                types = []  # results unused (e.g. a linalg op on memrefs printed with '-> ()')
            else:
                self.fail(f"op '{name}': {len(result_names)} result names for {len(types)} result types")
        for rn, t in zip(result_names, types):
            op.results.append(self.define(rn, t, op))
        return op

    def _fastmath(self) -> None:
        if self.accept_word("fastmath"):
            self.balanced("<", ">")

    def _typed_operand_list(self) -> list[Value]:
        """``(%a, %b : t1, t2)`` -> values (types checked for count only)."""
        self.expect("(")
        vals = []
        if self.accept(")"):
            return vals
        while True:
            vals.append(self.ssa_use())
            if not self.accept(","):
                break
        self.expect(":")
        n = 0
        while True:
            self.type()
            n += 1
            if not self.accept(","):
                break
        self.expect(")")
        if n != len(vals):
            self.fail("operand/type count mismatch")
        return vals

    def _linalg_structured(self, op: Operation) -> list:
        short = op.name.split(".", 1)[1]
        if self.peek("{"):
            op.attrs.update(self.attr_dict())
        while True:
            if self.accept_word("indexing_maps"):
                self.expect("=")
                op.attrs["indexing_maps"] = self.attr_value()
            elif self.accept_word("dimension"):
                self.expect("(")
                op.attrs["dimension"] = self.integer()
                self.expect(")")
            elif self.accept_word("kind"):
                self.expect("=")
                m = self.rx(re.compile(r"#linalg\.elementwise_kind<(\w+)>"))
                if not m:
                    self.fail("expected #linalg.elementwise_kind<...>")
                op.attrs["kind"] = m.group(1)
            else:
                break
        ins, outs = [], []
        if self.accept_word("ins"):
            ins = self._typed_operand_list()
        if self.accept_word("outs"):
            outs = self._typed_operand_list()
        else:
            self.fail(f"linalg.{short} without outs(...)")
        op.operands, op.n_ins = ins + outs, len(ins)
        while True:
            if self.accept_word("permutation"):
                self.expect("=")
                op.attrs["permutation"] = self.int_list()
            elif self.accept_word("dimensions"):
                self.expect("=")
                op.attrs["dimensions"] = self.int_list()
            elif self.accept_word("attrs"):
                self.expect("=")
                op.attrs.update(self.attr_dict())
            else:
                break
        if short == "generic":
            op.region = self._region()
        elif self.peek("{") and short in ("transpose", "broadcast"):
            self._region()  # printed form may carry the trivial yield region
        types = []
        if self.accept("->"):
            if self.accept("("):
                if not self.accept(")"):
                    while True:
                        types.append(self.type())
                        if self.accept(")"):
                            break
                        self.expect(",")
            else:
                types.append(self.type())
        return types

    def _region(self) -> Block:
        self.expect("{")
        block = Block()
        self.scopes.append({})
        if self.peek("^"):
            self.rx(re.compile(r"\^[A-Za-z0-9_]+"))
            if self.accept("("):
                if not self.accept(")"):
                    while True:
                        m = self.rx(_SSA)
                        self.expect(":")
                        block.args.append(self.define(m.group(0), self.type()))
                        if self.accept(")"):
                            break
                        self.expect(",")
            self.expect(":")
        while not self.accept("}"):
            block.ops.append(self.operation())
        self.scopes.pop()
        return block

    # -- individual custom-assembly ops -------------------------------------------------
    def _op_arith_constant(self, op):
        self.ws()
        if self.accept_word("dense"):
            self.fail("dense constants are not supported in payloads")
        if self.accept_word("true"):
            op.attrs["value"] = True
            return ["i1"]
        if self.accept_word("false"):
            op.attrs["value"] = False
            return ["i1"]
        m = self.rx(_NUMBER)
        if not m:
            self.fail("expected constant value")
        txt = m.group(0)
        self.expect(":")
        t = self.type()
        if t in ("f16", "bf16", "f32", "f64"):
            if txt.startswith("0x"):
                import struct

                # a hexadecimal float constant is the bit pattern at the type's own width
                bits = int(txt, 16)
                if t == "bf16":
                    op.attrs["value"] = struct.unpack("<f", struct.pack("<I", (bits & 0xFFFF) << 16))[0]
                elif t == "f16":
                    op.attrs["value"] = float(struct.unpack("<e", struct.pack("<H", bits & 0xFFFF))[0])
                elif t == "f64":
                    op.attrs["value"] = struct.unpack("<d", struct.pack("<Q", bits))[0]
                else:
                    op.attrs["value"] = struct.unpack("<f", struct.pack("<I", bits & 0xFFFFFFFF))[0]
            else:
                op.attrs["value"] = float(txt)
        else:
            op.attrs["value"] = int(txt, 0)
        return [t]

    def _op_tensor_empty(self, op):
        self.expect("(")
        self.expect(")")
        self.expect(":")
        return [self.type()]

    def _op_linalg_yield(self, op):
        if self.peek("%"):
            while True:
                op.operands.append(self.ssa_use())
                if not self.accept(","):
                    break
            self.expect(":")
            while True:
                self.type()
                if not self.accept(","):
                    break
        return []

    def _op_linalg_index(self, op):
        op.attrs["dim"] = self.integer()
        self.expect(":")
        return [self.type()]

    def _op_arith_cmpi(self, op):
        op.attrs["predicate"] = self.ident()
        self.expect(",")
        a = self.ssa_use()
        self.expect(",")
        b = self.ssa_use()
        self.expect(":")
        self.type()
        op.operands = [a, b]
        return ["i1"]

    def _op_complex_create(self, op):
        a = self.ssa_use()
        self.expect(",")
        b = self.ssa_use()
        self.expect(":")
        t = self.type()
        op.operands = [a, b]
        return [t]

    def _complex_part(self, op):
        a = self.ssa_use()
        self.expect(":")
        t = self.type()  # the operand's complex type
        op.operands = [a]
        return [t[len("complex<") : -1]]

    _op_complex_re = _complex_part
    _op_complex_im = _complex_part

    def _op_arith_cmpf(self, op):
        op.attrs["predicate"] = self.ident()
        self.expect(",")
        a = self.ssa_use()
        self.expect(",")
        b = self.ssa_use()
        self._fastmath()
        self.expect(":")
        self.type()
        op.operands = [a, b]
        return ["i1"]

    def _op_arith_select(self, op):
        c = self.ssa_use()
        self.expect(",")
        a = self.ssa_use()
        self.expect(",")
        b = self.ssa_use()
        self.expect(":")
        t = self.type()
        if self.accept(","):  # "i1, f32" form
            t = self.type()
        op.operands = [c, a, b]
        return [t]

    def _op_bufferization_to_tensor(self, op):
        op.operands = [self.ssa_use()]
        while True:
            if self.accept_word("restrict"):
                op.attrs["restrict"] = True
            elif self.accept_word("writable"):
                op.attrs["writable"] = True
            else:
                break
        self.expect(":")
        t = self.type()
        if self.accept_word("to"):
            return [self.type()]
        return [t.with_kind("tensor")]

    def _op_bufferization_materialize_in_destination(self, op):
        src = self.ssa_use()
        if not self.accept_word("in"):
            self.fail("expected 'in'")
        while True:
            if self.accept_word("restrict"):
                op.attrs["restrict"] = True
            elif self.accept_word("writable"):
                op.attrs["writable"] = True
            else:
                break
        dst = self.ssa_use()
        op.operands = [src, dst]
        self.expect(":")
        self.expect("(")
        self.type()
        self.expect(",")
        self.type()
        self.expect(")")
        self.expect("->")
        t = self.type()
        return [] if t == "()" else [t]

    def _reshape(self, op):
        op.operands = [self.ssa_use()]
        self.expect("[")
        groups = []
        if not self.accept("]"):
            while True:
                groups.append(self.int_list())
                if self.accept("]"):
                    break
                self.expect(",")
        op.attrs["reassociation"] = groups
        if self.accept_word("output_shape"):
            self.expect("[")
            shape = []
            if not self.accept("]"):
                while True:
                    shape.append(self.integer())
                    if self.accept("]"):
                        break
                    self.expect(",")
            op.attrs["output_shape"] = shape
        self.expect(":")
        self.type()
        if not self.accept_word("into"):
            self.fail("expected 'into'")
        return [self.type()]

    _op_memref_collapse_shape = _reshape
    _op_memref_expand_shape = _reshape
    _op_tensor_collapse_shape = _reshape
    _op_tensor_expand_shape = _reshape

    def _op_memref_transpose(self, op):
        op.operands = [self.ssa_use()]
        dims = [d.strip() for d in self.balanced("(", ")").split(",")]
        self.expect("->")
        res = [d.strip() for d in self.balanced("(", ")").split(",")]
        op.attrs["permutation"] = [dims.index(r) for r in res]
        self.expect(":")
        self.type()
        if not self.accept_word("to"):
            self.fail("expected 'to'")
        return [self.type()]

    def _alloc(self, op):
        while self.accept_word("host_shared") or self.accept_word("async"):
            pass
        if self.peek("["):
            self.balanced("[", "]")
        self.expect("(")
        self.expect(")")
        if self.peek("{"):
            self.attr_dict()
        self.expect(":")
        return [self.type()]

    _op_gpu_alloc = _alloc
    _op_memref_alloc = _alloc

    def _dealloc(self, op):
        while self.accept_word("async"):
            pass
        op.operands = [self.ssa_use()]
        self.expect(":")
        self.type()
        return []

    _op_gpu_dealloc = _dealloc
    _op_memref_dealloc = _dealloc

    def _op_gpu_memcpy(self, op):
        dst = self.ssa_use()
        self.expect(",")
        src = self.ssa_use()
        self.expect(":")
        self.type()
        self.expect(",")
        self.type()
        op.operands = [dst, src]
        return []

    def _op_memref_copy(self, op):
        src = self.ssa_use()
        self.expect(",")
        dst = self.ssa_use()
        self.expect(":")
        self.type()
        if not self.accept_word("to"):
            self.fail("expected 'to'")
        self.type()
        op.operands = [src, dst]
        return []

    def _return(self, op):
        if self.peek("%"):
            while True:
                op.operands.append(self.ssa_use())
                if not self.accept(","):
                    break
            self.expect(":")
            while True:
                self.type()
                if not self.accept(","):
                    break
        return []

    _op_return = _return
    _op_func_return = _return


def parse_mlir(text: str) -> PayloadModule:
    """MLIR text -> ``PayloadModule``. Raises ``ValueError`` for anything outside the subset."""
    if not isinstance(text, str) or not text.strip():
        raise ValueError("empty MLIR payload")
    return _Parser(text).module()
