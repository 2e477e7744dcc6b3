"""A ``torch.compile`` backend in the shape of the reference's
(lighthouse/ingress/torch/compile.py:42-151 ``TorchMemoryManager`` / ``JITFunction``, :154-411
``MLIRBackend``, :414-487 ``cpu_backend`` / ``gpu_backend``).

The reference imports the FX graph into MLIR with torch-mlir, moves the results into trailing
buffer arguments (:288-338) and JIT-compiles it. torch-mlir is not part of this backend, so the
FX graph Dynamo hands over is pattern-matched directly: linear / matmul, activations, residual
and bias adds, layer norm, softmax, scaled-dot-product attention and the view operators
between them become the operators of a ``Plan`` (the same operator records the MLIR payload
recogniser produces), the epilogue fusion passes run on it, and a ``JITFunction`` executes it
on the CUDA kernels with the caller's torch tensors passed by pointer. Calling convention as
in the reference: inputs in placeholder order, result buffers appended last, results returned
as a list. A graph with anything else in it is a ``ValueError``: there is no eager fallback.
"""

from __future__ import annotations

import math
import operator
from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np
import torch

from ...payload.lower import compact_temps, fuse_gemm_epilogues, fuse_norm_cast
from ...plan import ArgSpec, Plan, PView

_DTYPE_NAMES = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16", torch.int32: "i32", torch.int64: "i64"}


class UnsupportedGraph(ValueError):
    """The FX graph holds an operator (or a shape / dtype) this backend has no kernel for."""


@dataclass
class BufferMetadata:
    """Shape, dtype and device of a result buffer (compile.py:34-40 of the reference)."""

    shape: list[int]
    dtype: torch.dtype
    device: torch.device


def _target_name(target) -> str:
    if isinstance(target, str):
        return target
    name = getattr(target, "__name__", None) or str(target)
    return name


class _Importer:
    """Walks the graph once; every tensor value is a ``PView`` (views cost nothing)."""

    def __init__(self, gm: torch.fx.GraphModule, example_inputs: Sequence[torch.Tensor], entry: str):
        self.gm = gm
        self.entry = entry
        placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
        if len(placeholders) != len(example_inputs):
            raise UnsupportedGraph(f"graph takes {len(placeholders)} inputs, {len(example_inputs)} examples given")
        args = []
        for node, t in zip(placeholders, example_inputs):
            if not isinstance(t, torch.Tensor):
                raise UnsupportedGraph(f"input '{node.name}' is not a tensor")
            if t.dtype not in _DTYPE_NAMES:
                raise UnsupportedGraph(f"input '{node.name}' has dtype {t.dtype}")
            args.append(ArgSpec(tuple(int(d) for d in t.shape), _DTYPE_NAMES[t.dtype], node.name))
        self.n_inputs = len(args)
        self.device = example_inputs[0].device if example_inputs else torch.device("cpu")
        # result buffers are appended once the output node is known
        self.input_args = args
        self.values: dict = {}
        self.ops: list = []  # deferred emitters, replayed on the final Plan

    # -- helpers -----------------------------------------------------------------------
    def _val(self, x):
        return self.values[x] if isinstance(x, torch.fx.Node) else x

    def _tensor(self, node, what: str) -> PView:
        v = self._val(node)
        if not isinstance(v, PView):
            raise UnsupportedGraph(f"{what}: expected a tensor, got {type(v).__name__}")
        return v

    def _contiguous(self, p: Plan, v: PView) -> PView:
        if v.is_contiguous():
            return v
        out = p.temp(v.shape, v.dtype)
        p.elementwise("copy", out, v)
        return out

    # -- operators ---------------------------------------------------------------------
    def _linear(self, p: Plan, x: PView, w: PView, b) -> PView:
        if w.rank != 2 or x.shape[-1] != w.shape[1]:
            raise UnsupportedGraph(f"linear: input {x.shape} x weight {w.shape}")
        lead = x.shape[:-1]
        try:
            x2 = x.reshape((math.prod(lead), x.shape[-1]))
        except ValueError:
            x2 = self._contiguous(p, x).reshape((math.prod(lead), x.shape[-1]))
        out = p.temp((x2.shape[0], w.shape[0]), x.dtype)
        p.gemm(out, x2, w.t(), bias=b)
        return out.reshape(tuple(lead) + (w.shape[0],))

    def _matmul(self, p: Plan, a: PView, b: PView) -> PView:
        if a.rank == 2 and b.rank == 2 and a.shape[1] == b.shape[0]:
            out = p.temp((a.shape[0], b.shape[1]), a.dtype)
            p.gemm(out, a, b)
            return out
        if a.rank == 3 and b.rank == 3 and a.shape[0] == b.shape[0] and a.shape[2] == b.shape[1]:
            out = p.temp((a.shape[0], a.shape[1], b.shape[2]), a.dtype)
            p.gemm(out, a, b)
            return out
        if a.rank > 2 and b.rank == 2 and a.shape[-1] == b.shape[0]:
            a2 = self._contiguous(p, a).reshape((math.prod(a.shape[:-1]), a.shape[-1]))
            out = p.temp((a2.shape[0], b.shape[1]), a.dtype)
            p.gemm(out, a2, b)
            return out.reshape(tuple(a.shape[:-1]) + (b.shape[1],))
        raise UnsupportedGraph(f"matmul of shapes {a.shape} and {b.shape}")

    def _act(self, p: Plan, x: PView, act: str) -> PView:
        out = p.temp(x.shape, x.dtype)
        p.elementwise("act", out, x, act=act)
        return out

    def _binary(self, p: Plan, kind: str, a, b) -> PView:
        if not isinstance(a, PView) and isinstance(b, PView) and kind in ("add", "mul"):
            a, b = b, a
        if isinstance(a, PView) and isinstance(b, (int, float)):
            if kind == "mul":
                out = p.temp(a.shape, a.dtype)
                p.elementwise("scale", out, a, scalar=float(b))
                return out
            raise UnsupportedGraph(f"tensor {kind} scalar")
        if not (isinstance(a, PView) and isinstance(b, PView)):
            raise UnsupportedGraph(f"{kind} of non-tensors")
        if a.shape != b.shape:
            if b.rank == 1 and b.shape[0] == a.shape[-1]:  # row vector (a bias) over every row
                b = b.broadcast_to(a.shape, set(range(a.rank - 1)))
            elif a.rank == 1 and a.shape[0] == b.shape[-1] and kind in ("add", "mul"):
                a, b = b, a.broadcast_to(b.shape, set(range(b.rank - 1)))
            else:
                raise UnsupportedGraph(f"{kind} of shapes {a.shape} and {b.shape}")
        out = p.temp(a.shape, a.dtype)
        p.elementwise(kind, out, a, b)
        return out

    def _layer_norm(self, p: Plan, x: PView, normalized_shape, weight, bias, eps) -> PView:
        if len(tuple(normalized_shape)) != 1 or int(tuple(normalized_shape)[0]) != x.shape[-1]:
            raise UnsupportedGraph("layer_norm over more than the last dimension")
        x2 = self._contiguous(p, x).reshape((math.prod(x.shape[:-1]), x.shape[-1]))
        out = p.temp(x2.shape, x.dtype)
        p.layernorm(out, x2, weight, bias, float(eps))
        return out.reshape(x.shape)

    def _softmax(self, p: Plan, x: PView, dim) -> PView:
        if dim not in (-1, x.rank - 1):
            raise UnsupportedGraph("softmax over a dimension other than the last")
        x2 = self._contiguous(p, x).reshape((math.prod(x.shape[:-1]), x.shape[-1]))
        out = p.temp(x2.shape, x.dtype)
        p.softmax(out, x2)
        return out.reshape(x.shape)

    def _sdpa(self, p: Plan, q: PView, k: PView, v: PView, kw: dict) -> PView:
        if kw.get("attn_mask") is not None or kw.get("dropout_p", 0.0) not in (0, 0.0) or kw.get("enable_gqa", False):
            raise UnsupportedGraph("scaled_dot_product_attention with a mask tensor, dropout or enable_gqa")
        if q.rank not in (3, 4):
            raise UnsupportedGraph(f"attention on rank-{q.rank} tensors")
        scale = kw.get("scale")
        scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        out = p.temp(q.shape, q.dtype)
        p.attention(out, q, k, v, scale, bool(kw.get("is_causal", False)))
        return out

    @staticmethod
    def _index(x: PView, index) -> PView:
        """Basic indexing (ints, slices, Ellipsis) as a view."""
        index = index if isinstance(index, tuple) else (index,)
        if any(i is None or isinstance(i, (PView, torch.Tensor, list)) for i in index):
            raise UnsupportedGraph("indexing with None or with tensors")
        n_explicit = sum(1 for i in index if i is not Ellipsis)
        expanded = []
        for i in index:
            expanded.extend([slice(None)] * (x.rank - n_explicit) if i is Ellipsis else [i])
        expanded.extend([slice(None)] * (x.rank - len(expanded)))
        shape, strides, offset = [], [], x.offset
        for d, i in enumerate(expanded):
            if isinstance(i, int):
                i = i % x.shape[d]
                offset += i * x.strides[d]
            else:
                start, stop, step = i.indices(x.shape[d])
                if step <= 0:
                    raise UnsupportedGraph("slices with a non-positive step")
                shape.append(max(0, -(-(stop - start) // step)))
                strides.append(x.strides[d] * step)
                offset += start * x.strides[d]
        return PView(x.slot, tuple(shape), tuple(strides), x.dtype, offset)

    # -- the walk ----------------------------------------------------------------------
    def run(self) -> tuple[Plan, list[BufferMetadata], int]:
        output_node = next(n for n in self.gm.graph.nodes if n.op == "output")
        outs = output_node.args[0]
        outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
        # first pass on a scratch plan to learn the result shapes, second with result arguments
        plan = Plan(self.entry, list(self.input_args))
        self._walk(plan)
        result_views = [self._tensor(o, "graph output") for o in outs]
        results = [BufferMetadata(list(v.shape), {n: t for t, n in _DTYPE_NAMES.items()}[v.dtype], self.device) for v in result_views]
        final = Plan(self.entry, list(self.input_args) + [ArgSpec(tuple(v.shape), v.dtype, f"result{i}") for i, v in enumerate(result_views)])
        self.values = {}
        self._walk(final, shift=len(result_views))
        nargs = len(final.args)
        for i, o in enumerate(outs):
            v = self._tensor(o, "graph output")
            dst = final.arg(self.n_inputs + i)
            producers = [op for op in final.ops if op.operands[0] is not None and op.operands[0].slot == v.slot]
            if v.slot >= nargs and v.offset == 0 and v.is_contiguous() and len(producers) == 1 and producers[0].operands[0].shape == v.shape:
                # the value is a whole temporary: let its producer (and its readers) use the result buffer
                old = v.slot
                for op in final.ops:
                    op.operands = [None if w is None else (PView(dst.slot, w.shape, w.strides, w.dtype, w.offset) if w.slot == old else w) for w in op.operands]
            else:
                final.elementwise("copy", dst, v)
        fuse_gemm_epilogues(final)
        fuse_norm_cast(final)
        compact_temps(final)
        return final, results, len(outs)

    def _walk(self, p: Plan, shift: int = 0) -> None:
        """``shift`` result arguments follow the inputs, so temporaries start that much later;
        nothing else changes between the two passes."""
        index = 0
        for node in self.gm.graph.nodes:
            if node.op == "placeholder":
                self.values[node] = p.arg(index)
                index += 1
            elif node.op == "get_attr":
                raise UnsupportedGraph(f"constant tensor '{node.target}' embedded in the graph (parameters must be graph inputs)")
            elif node.op in ("call_function", "call_method"):
                self.values[node] = self._call(p, node)
            elif node.op == "output":
                pass
            else:
                raise UnsupportedGraph(f"node kind '{node.op}'")

    def _call(self, p: Plan, node):
        name = _target_name(node.target)
        a = [self._val(x) for x in node.args]
        kw = {k: self._val(v) for k, v in node.kwargs.items()}
        method = node.op == "call_method"
        if name == "linear":
            return self._linear(p, self._tensor(node.args[0], name), self._tensor(node.args[1], name), a[2] if len(a) > 2 else kw.get("bias"))
        if name in ("matmul", "mm", "bmm") or node.target is operator.matmul:
            return self._matmul(p, self._tensor(node.args[0], name), self._tensor(node.args[1], name))
        if name in ("relu", "relu_"):
            return self._act(p, self._tensor(node.args[0], name), "relu")
        if name == "gelu":
            approx = kw.get("approximate", a[1] if len(a) > 1 else "none")
            return self._act(p, self._tensor(node.args[0], name), "gelu_tanh" if approx == "tanh" else "gelu")
        if name == "silu":
            return self._act(p, self._tensor(node.args[0], name), "silu")
        if name == "sigmoid":
            return self._act(p, self._tensor(node.args[0], name), "sigmoid")
        if name in ("add", "iadd", "add_") or node.target is operator.add:
            if kw.get("alpha", 1) != 1:
                raise UnsupportedGraph("add with alpha")
            return self._binary(p, "add", a[0], a[1])
        if name in ("mul", "imul") or node.target is operator.mul:
            return self._binary(p, "mul", a[0], a[1])
        if name == "sub" or node.target is operator.sub:
            return self._binary(p, "sub", a[0], a[1])
        if name == "layer_norm":
            x = self._tensor(node.args[0], name)
            return self._layer_norm(p, x, a[1], a[2] if len(a) > 2 else kw.get("weight"), a[3] if len(a) > 3 else kw.get("bias"), a[4] if len(a) > 4 else kw.get("eps", 1e-5))
        if name == "rms_norm":
            x = self._tensor(node.args[0], name)
            shape = tuple(a[1])
            weight = a[2] if len(a) > 2 else kw.get("weight")
            eps = a[3] if len(a) > 3 else kw.get("eps")
            if len(shape) != 1 or int(shape[0]) != x.shape[-1]:
                raise UnsupportedGraph("rms_norm over more than the last dimension")
            x2 = self._contiguous(p, x).reshape((math.prod(x.shape[:-1]), x.shape[-1]))
            out = p.temp(x2.shape, x.dtype)
            p.rmsnorm(out, x2, weight, float(eps) if eps is not None else float(torch.finfo({n: t for t, n in _DTYPE_NAMES.items()}[x.dtype]).eps))
            return out.reshape(x.shape)
        if name == "embedding":
            ids, table = self._tensor(node.args[0], name), self._tensor(node.args[1], name)
            if ids.dtype not in ("i32", "i64") or table.rank != 2 or any(v is not None for v in a[2:3]) or kw.get("padding_idx") is not None:
                raise UnsupportedGraph("embedding with a padding index or non-integer ids")
            flat = self._contiguous(p, ids).reshape((ids.numel,))
            out = p.temp((ids.numel, table.shape[1]), table.dtype)
            p.embedding(out, flat, table, None, 0)
            return out.reshape(tuple(ids.shape) + (table.shape[1],))
        if name == "softmax":
            x = self._tensor(node.args[0], name)
            dim = a[1] if len(a) > 1 else kw.get("dim", -1)
            if kw.get("dtype") is not None or (len(a) > 3 and a[3] is not None):
                raise UnsupportedGraph("softmax with a dtype argument")
            return self._softmax(p, x, dim)
        if name == "scaled_dot_product_attention":
            q, k, v = (self._tensor(n, name) for n in node.args[:3])
            names = ["attn_mask", "dropout_p", "is_causal", "scale", "enable_gqa"]
            kw = {**dict(zip(names, a[3:])), **kw}
            return self._sdpa(p, q, k, v, kw)
        # views
        if name == "getitem" or node.target is operator.getitem:
            base = a[0]
            if isinstance(base, (tuple, list)):
                return base[a[1]]
            return self._index(self._tensor(node.args[0], name), a[1])
        if name in ("split", "chunk"):
            x = self._tensor(node.args[0], name)
            dim = (a[2] if len(a) > 2 else kw.get("dim", 0)) % x.rank
            if name == "chunk":
                size = -(-x.shape[dim] // int(a[1]))
            else:
                size = a[1] if len(a) > 1 else kw.get("split_size_or_sections", kw.get("split_size"))
            if not isinstance(size, int):
                raise UnsupportedGraph("split into sections of different sizes")
            return tuple(x.slice(dim, s0, min(size, x.shape[dim] - s0)) for s0 in range(0, x.shape[dim], size))
        if name in ("view", "reshape", "_unsafe_view"):
            x = self._tensor(node.args[0], name)
            shape = a[1] if len(a) == 2 and isinstance(a[1], (tuple, list, torch.Size)) else a[1:]
            shape = [int(d) for d in shape]
            if -1 in shape:
                known = -math.prod(shape)
                shape[shape.index(-1)] = x.numel // known
            try:
                return x.reshape(shape)
            except ValueError:
                if name == "view":
                    raise UnsupportedGraph(f"view of a non-contiguous tensor to {shape}")
                return self._contiguous(p, x).reshape(shape)
        if name == "flatten":
            x = self._tensor(node.args[0], name)
            start = (a[1] if len(a) > 1 else kw.get("start_dim", 0)) % x.rank
            end = (a[2] if len(a) > 2 else kw.get("end_dim", -1)) % x.rank
            shape = x.shape[:start] + (math.prod(x.shape[start : end + 1]),) + x.shape[end + 1 :]
            try:
                return x.reshape(shape)
            except ValueError:
                return self._contiguous(p, x).reshape(shape)
        if name == "transpose":
            x = self._tensor(node.args[0], name)
            perm = list(range(x.rank))
            d0, d1 = a[1] % x.rank, a[2] % x.rank
            perm[d0], perm[d1] = perm[d1], perm[d0]
            return x.permute(perm)
        if name == "permute":
            x = self._tensor(node.args[0], name)
            perm = a[1] if len(a) == 2 and isinstance(a[1], (tuple, list)) else a[1:]
            return x.permute([int(d) % x.rank for d in perm])
        if name == "t" and method:
            return self._tensor(node.args[0], name).t()
        if name == "contiguous":
            return self._contiguous(p, self._tensor(node.args[0], name))
        if name in ("detach", "clone") and method:
            return self._tensor(node.args[0], name)
        if name in ("to", "type") and method:
            x = self._tensor(node.args[0], name)
            dt = next((v for v in list(a[1:]) + list(kw.values()) if isinstance(v, torch.dtype)), None)
            if dt is None or _DTYPE_NAMES.get(dt) == x.dtype:
                return x
            if dt not in _DTYPE_NAMES:
                raise UnsupportedGraph(f"cast to {dt}")
            out = p.temp(x.shape, _DTYPE_NAMES[dt])
            p.elementwise("copy", out, x)
            return out
        raise UnsupportedGraph(f"no kernel for '{name}' ({node.op})")


def import_fx_graph(gm: torch.fx.GraphModule, example_inputs: Sequence[torch.Tensor], entry_func: str = "main") -> tuple[Plan, list[BufferMetadata], int]:
    """FX graph -> (plan with the result buffers as trailing arguments, their metadata, count)."""
    return _Importer(gm, example_inputs, entry_func).run()


class JITFunction:
    """The compiled callable (compile.py:51-151 of the reference): owns the module, allocates
    the result buffers, passes inputs followed by result buffers, returns the results."""

    def __init__(self, plan: Plan, results: list[BufferMetadata], entry_func: str = "main", n_outputs: int | None = None, context=None):
        self.plan = plan
        self.results = results
        self.entry_func = entry_func
        self.n_outputs = n_outputs if n_outputs is not None else len(results)
        self._ctx = context
        self._session = None

    def _ensure_session(self, device: torch.device):
        if self._session is None:
            from ...context import CudaContext
            from ...workloads.session import PlanSession

            if device.type != "cuda":
                raise RuntimeError("this backend runs on CUDA tensors only (there is no CPU path)")
            if self._ctx is None:
                self._ctx = CudaContext(device.index if device.index is not None else torch.cuda.current_device())
            self._session = PlanSession(self.plan, ctx=self._ctx)
        return self._session

    def _generate_input_args(self, *args: torch.Tensor) -> tuple[list[torch.Tensor], list[torch.Tensor]]:
        device = args[0].device if args else self.results[0].device
        outs = [torch.empty(r.shape, dtype=r.dtype, device=device) for r in self.results]
        all_tensors = [a.detach().contiguous() for a in args]
        all_tensors.extend(outs)
        return all_tensors, outs

    def __call__(self, *args: torch.Tensor) -> list[torch.Tensor]:
        all_tensors, outs = self._generate_input_args(*args)
        session = self._ensure_session(all_tensors[0].device)
        self._ctx.use_torch_stream()  # ordered with the caller's torch work, no synchronisation
        session.run(all_tensors)
        return outs[len(self.results) - self.n_outputs :]

    def benchmark(self, *args: torch.Tensor, nruns: int = 500, nwarmup: int = 500) -> np.ndarray:
        """Seconds per run; parameters first, then inputs, as the graph takes them."""
        all_tensors, _ = self._generate_input_args(*args)
        session = self._ensure_session(all_tensors[0].device)
        self._ctx.use_torch_stream()
        return session.benchmark(all_tensors, nruns=nruns, nwarmup=nwarmup)


class CudaBackend:
    """``torch.compile(model, backend=CudaBackend(...))`` (``MLIRBackend``, compile.py:154-411)."""

    def __init__(self, device: torch.device, fn_compile: Callable[[Plan], Plan] | None = None, entry_func: str = "main", context=None):
        self.device = device
        self.fn_compile = fn_compile
        self.entry_func = entry_func
        self.context = context
        self._last_jit_function: JITFunction | None = None

    @staticmethod
    def is_symbolic(t) -> bool:
        return isinstance(t, torch.Tensor) and any(isinstance(d, torch.SymInt) for d in t.shape)

    def __call__(self, model: torch.fx.GraphModule, example_inputs: list[torch.Tensor]) -> JITFunction:
        if any(self.is_symbolic(t) for t in example_inputs):
            raise ValueError("Dynamic shapes are not supported - consider using 'torch.compile(..., dynamic=False)'")
        plan, results, n_out = import_fx_graph(model, example_inputs, self.entry_func)
        if self.fn_compile is not None:
            plan = self.fn_compile(plan)
        jit_fn = JITFunction(plan, results, entry_func=self.entry_func, n_outputs=n_out, context=self.context)
        self._last_jit_function = jit_fn
        return jit_fn


def gpu_backend(fn_compile: Callable[[Plan], Plan] | None = None, device: torch.device | None = None, entry_func: str = "main", context=None) -> CudaBackend:
    """The reference's ``gpu_backend(fn_compile, device, ...)`` (compile.py:455-487): here
    ``fn_compile`` is an optional hook over the plan instead of an MLIR lowering function."""
    device = device if device is not None else torch.device("cuda")
    assert device.type == "cuda", "Expected a CUDA device"
    return CudaBackend(device, fn_compile, entry_func=entry_func, context=context)
