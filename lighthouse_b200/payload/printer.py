"""Prints a ``PayloadModule`` as MLIR text in the custom assembly the upstream printer
uses for these ops, so that what the builders in ``generators.py`` produce can be fed to
any tool that reads MLIR — and back through ``parser.parse_mlir``."""

from __future__ import annotations

from .ir import AffineMap, Block, Func, Operation, PayloadModule, ShapedType


# bit patterns of NaN, +inf, -inf at each float type's width (MLIR reads a hexadecimal float
# constant as the bits of its own type)
_SPECIAL_BITS = {"f32": ("0x7FC00000", "0x7F800000", "0xFF800000"), "bf16": ("0x7FC0", "0x7F80", "0xFF80"),
                 "f16": ("0x7E00", "0x7C00", "0xFC00"), "f64": ("0x7FF8000000000000", "0x7FF0000000000000", "0xFFF0000000000000")}


def _fmt_float(v: float, t: str = "f32") -> str:
    if v != v:
        return _SPECIAL_BITS[t][0]
    if v in (float("inf"), float("-inf")):
        return _SPECIAL_BITS[t][1 if v > 0 else 2]
    s = f"{v:.6e}"
    if float(s) != v:
        s = repr(float(v))
        if "e" not in s and "." not in s:
            s += ".0"
    return s


def _types(vals) -> str:
    return ", ".join(str(v.type) for v in vals)


def _names(vals) -> str:
    return ", ".join(v.name for v in vals)


def _attr(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, AffineMap):
        return str(v)
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(_attr(x) for x in v) + "]"
    if isinstance(v, str):
        return f'"{v}"'
    return str(v)


def _print_op(op: Operation, ind: str, out: list[str]) -> None:
    res = f"{_names(op.results)} = " if op.results else ""
    n = op.name
    if n == "arith.constant":
        t = op.results[0].type
        val = op.attrs["value"]
        txt = _fmt_float(float(val), str(t)) if t in ("f16", "bf16", "f32", "f64") else str(int(val))
        out.append(f"{ind}{res}arith.constant {txt} : {t}")
    elif n == "tensor.empty":
        out.append(f"{ind}{res}tensor.empty() : {op.results[0].type}")
    elif n == "complex.create":
        out.append(f"{ind}{res}complex.create {_names(op.operands)} : {op.results[0].type}")
    elif n in ("complex.re", "complex.im"):
        out.append(f"{ind}{res}{n} {op.operands[0].name} : {op.operands[0].type}")
    elif n == "complex.mul":
        out.append(f"{ind}{res}complex.mul {_names(op.operands)} : {op.results[0].type}")
    elif n == "arith.cmpi":
        out.append(f"{ind}{res}arith.cmpi {op.attrs['predicate']}, {_names(op.operands)} : {op.operands[0].type}")
    elif n.startswith("linalg.") and n not in ("linalg.yield", "linalg.index"):
        head = f"{ind}{res}{n}"
        if n == "linalg.generic":
            maps = "[" + ", ".join(str(m) for m in op.attrs["indexing_maps"]) + "]"
            iters = "[" + ", ".join(f'"{i}"' for i in op.attrs["iterator_types"]) + "]"
            head += f" {{indexing_maps = {maps}, iterator_types = {iters}}}"
        if n == "linalg.contract":
            head += " indexing_maps = [" + ", ".join(str(m) for m in op.attrs["indexing_maps"]) + "]"
        if n == "linalg.elementwise":
            head += f" kind=#linalg.elementwise_kind<{op.attrs['kind']}>"
        if n == "linalg.softmax":
            head += f" dimension({op.attrs['dimension']})"
        if op.ins:
            head += f" ins({_names(op.ins)} : {_types(op.ins)})"
        head += f" outs({_names(op.outs)} : {_types(op.outs)})"
        if "permutation" in op.attrs:
            head += f" permutation = {_attr(op.attrs['permutation'])}"
        if "dimensions" in op.attrs:
            head += f" dimensions = {_attr(op.attrs['dimensions'])}"
        tail = f" -> {_types(op.results)}" if op.results else ""
        if op.region is not None:
            out.append(head + " {")
            _print_block(op.region, ind + "  ", out, label=True)
            out.append(f"{ind}}}{tail}")
        else:
            out.append(head + tail)
    elif n == "linalg.index":
        out.append(f"{ind}{res}linalg.index {op.attrs['dim']} : index")
    elif n == "linalg.yield":
        out.append(f"{ind}linalg.yield {_names(op.operands)} : {_types(op.operands)}" if op.operands else f"{ind}linalg.yield")
    elif n == "bufferization.to_tensor":
        flags = "".join(f" {k}" for k in ("restrict", "writable") if op.attrs.get(k))
        out.append(f"{ind}{res}bufferization.to_tensor {op.operands[0].name}{flags} : {op.operands[0].type} to {op.results[0].type}")
    elif n == "bufferization.materialize_in_destination":
        flags = "".join(f"{k} " for k in ("restrict", "writable") if op.attrs.get(k))
        src, dst = op.operands
        rt = str(op.results[0].type) if op.results else "()"
        out.append(f"{ind}{res}bufferization.materialize_in_destination {src.name} in {flags}{dst.name} : ({src.type}, {dst.type}) -> {rt}")
    elif n in ("memref.collapse_shape", "memref.expand_shape", "tensor.collapse_shape", "tensor.expand_shape"):
        line = f"{ind}{res}{n} {op.operands[0].name} {_attr(op.attrs['reassociation'])}"
        if "output_shape" in op.attrs:
            line += f" output_shape {_attr(op.attrs['output_shape'])}"
        out.append(f"{line} : {op.operands[0].type} into {op.results[0].type}")
    elif n == "memref.transpose":
        perm = op.attrs["permutation"]
        dims = ", ".join(f"d{i}" for i in range(len(perm)))
        res_dims = ", ".join(f"d{i}" for i in perm)
        out.append(f"{ind}{res}memref.transpose {op.operands[0].name} ({dims}) -> ({res_dims}) : {op.operands[0].type} to {op.results[0].type}")
    elif n in ("gpu.alloc", "memref.alloc"):
        out.append(f"{ind}{res}{n} () : {op.results[0].type}" if n == "gpu.alloc" else f"{ind}{res}{n}() : {op.results[0].type}")
    elif n in ("gpu.dealloc", "memref.dealloc"):
        out.append(f"{ind}{n} {op.operands[0].name} : {op.operands[0].type}")
    elif n in ("return", "func.return"):
        out.append(f"{ind}return {_names(op.operands)} : {_types(op.operands)}" if op.operands else f"{ind}return")
    elif n in ("arith.truncf", "arith.extf", "arith.sitofp", "arith.index_cast"):
        out.append(f"{ind}{res}{n} {op.operands[0].name} : {op.operands[0].type} to {op.results[0].type}")
    elif n == "arith.cmpf":
        out.append(f"{ind}{res}arith.cmpf {op.attrs['predicate']}, {_names(op.operands)} : {op.operands[0].type}")
    elif n == "arith.select":
        out.append(f"{ind}{res}arith.select {_names(op.operands)} : {op.results[0].type}")
    elif n.startswith("arith.") or n.startswith("math."):
        out.append(f"{ind}{res}{n} {_names(op.operands)} : {op.results[0].type}")
    else:
        raise ValueError(f"cannot print op '{n}'")


def _print_block(block: Block, ind: str, out: list[str], label: bool) -> None:
    if label:
        args = ", ".join(f"{a.name}: {a.type}" for a in block.args)
        out.append(f"{ind[:-2]}^bb0({args}):")
    for op in block.ops:
        _print_op(op, ind, out)


def print_func(fn: Func, ind: str = "  ") -> list[str]:
    args = ", ".join(f"{a.name}: {a.type}" for a in fn.args)
    res = ""
    if fn.result_types:
        res = " -> " + (str(fn.result_types[0]) if len(fn.result_types) == 1 else "(" + ", ".join(map(str, fn.result_types)) + ")")
    attrs = {k: v for k, v in fn.attrs.items() if k != "visibility"}
    attr_txt = ""
    if attrs:
        attr_txt = " attributes {" + ", ".join(k if v is True else f"{k} = {_attr(v)}" for k, v in attrs.items()) + "}"
    out = [f"{ind}func.func @{fn.name}({args}){res}{attr_txt} {{"]
    _print_block(fn.body, ind + "  ", out, label=False)
    out.append(f"{ind}}}")
    return out


def print_module(pm: PayloadModule) -> str:
    out = ["module {"]
    for fn in pm.funcs.values():
        if fn.body is not None:
            out.extend(print_func(fn))
    out.append("}")
    return "\n".join(out) + "\n"
