"""Plans: the recognised form of a payload function.

A plan is what the CUDA dispatch stage produces from a payload module and what
the native library executes (``lh_module_t``): numbered buffer slots — the entry
function's arguments in signature order, then temporaries — and a list of
operator records whose operands are strided views into those slots. It plays the
role the lowered LLVM module plays for the reference's ``Runner``
(lighthouse/execution/runner.py:129-137): the thing that is handed to the
execution engine.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field

from . import _native as N

ACT_CODES = {
    "none": N.ACT_NONE,
    "relu": N.ACT_RELU,
    "gelu": N.ACT_GELU_ERF,
    "gelu_erf": N.ACT_GELU_ERF,
    "gelu_tanh": N.ACT_GELU_TANH,
    "silu": N.ACT_SILU,
    "sigmoid": N.ACT_SIGMOID,
}
EW_CODES = {
    "copy": N.EW_COPY,
    "add": N.EW_ADD,
    "mul": N.EW_MUL,
    "act": N.EW_ACT,
    "add_act": N.EW_ADD_ACT,
    "silu_mul": N.EW_SILU_MUL,
    "scale": N.EW_SCALE,
    "fill": N.EW_FILL,
    "sub": N.EW_SUB,
    "max": N.EW_MAX,
}


def dtype_bytes(dtype: str) -> int:
    return N.DTYPE_SIZE[N.DTYPE_FROM_NAME[dtype]]


@dataclass(frozen=True)
class PView:
    """A strided view into buffer slot ``slot`` (strides and offset in elements)."""

    slot: int
    shape: tuple[int, ...]
    strides: tuple[int, ...]
    dtype: str
    offset: int = 0

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        return math.prod(self.shape)

    def is_contiguous(self) -> bool:
        expect = 1
        for d, s in zip(reversed(self.shape), reversed(self.strides)):
            if d != 1 and s != expect:
                return False
            expect *= d
        return True

    # -- view algebra (no data movement) ------------------------------------------
    def permute(self, perm) -> "PView":
        return PView(self.slot, tuple(self.shape[p] for p in perm), tuple(self.strides[p] for p in perm), self.dtype, self.offset)

    def t(self) -> "PView":
        perm = list(range(self.rank))
        perm[-1], perm[-2] = perm[-2], perm[-1]
        return self.permute(perm)

    def reshape(self, shape) -> "PView":
        """Reshape of a contiguous view, or any reshape expressible by merging/splitting
        adjacent dims whose strides nest (memref.collapse_shape / expand_shape)."""
        shape = tuple(int(d) for d in shape)
        if math.prod(shape) != self.numel:
            raise ValueError(f"cannot reshape {self.shape} to {shape}")
        if self.is_contiguous():
            return PView(self.slot, shape, tuple(N.contiguous_strides(shape)), self.dtype, self.offset)
        # general case: merge maximal nested groups, then split them
        groups = []  # (size, stride) of merged dims, outermost first
        for d, s in zip(self.shape, self.strides):
            if d == 1:
                continue
            if groups and groups[-1][1] == s * d:
                groups[-1] = (groups[-1][0] * d, s)
            else:
                groups.append((d, s))
        new_strides = []
        gi, remaining = 0, groups[0][0] if groups else 1
        for d in shape:
            if d == 1:
                new_strides.append(1)
                continue
            if gi >= len(groups) or remaining % d:
                raise ValueError(f"reshape {self.shape}/{self.strides} -> {shape} needs a copy")
            remaining //= d
            new_strides.append(groups[gi][1] * remaining)
            if remaining == 1:
                gi += 1
                remaining = groups[gi][0] if gi < len(groups) else 1
        return PView(self.slot, shape, tuple(new_strides), self.dtype, self.offset)

    def slice(self, dim: int, start: int, length: int) -> "PView":
        if start < 0 or start + length > self.shape[dim]:
            raise ValueError("slice out of range")
        shape = list(self.shape)
        shape[dim] = length
        return PView(self.slot, tuple(shape), self.strides, self.dtype, self.offset + start * self.strides[dim])

    def broadcast_to(self, shape, dims_added) -> "PView":
        """linalg.broadcast: ``dims_added`` are the output dims that do not exist in the input."""
        it = iter(range(self.rank))
        new_shape, new_strides = [], []
        for d in range(len(shape)):
            if d in dims_added:
                new_shape.append(shape[d])
                new_strides.append(0)
            else:
                i = next(it)
                new_shape.append(self.shape[i])
                new_strides.append(self.strides[i])
        return PView(self.slot, tuple(new_shape), tuple(new_strides), self.dtype, self.offset)

    def to_native(self) -> N.View:
        v = N.View()
        v.slot = self.slot
        v.rank = self.rank
        v.dtype = N.DTYPE_FROM_NAME[self.dtype]
        v.offset = self.offset
        for i in range(self.rank):
            v.shape[i] = self.shape[i]
            v.strides[i] = self.strides[i]
        return v


@dataclass
class PlanOp:
    kind: str  # one of the keys of _KIND_CODES below
    operands: list  # PView | None, in the order lh_b200.h documents
    attrs: dict = field(default_factory=dict)

    def flops(self) -> int:
        """Algorithmic flops with the reference's conventions (examples/xegpu/matmul.py:52-64,
        examples/xegpu/fused_attention.py:38-43)."""
        if self.kind in ("gemm", "gemm_rope"):
            a, b = self.operands[1], self.operands[2]
            batch = a.shape[0] if a.rank == 3 else 1
            return 2 * batch * a.shape[-2] * a.shape[-1] * b.shape[-1]
        if self.kind == "attention":
            q, k = self.operands[1], self.operands[2]
            f = 4 * math.prod(q.shape[:-2]) * q.shape[-2] * k.shape[-2] * q.shape[-1]
            return f // 2 if self.attrs.get("causal") else f
        return 0


_KIND_CODES = {
    "gemm": N.OP_GEMM,
    "attention": N.OP_ATTENTION,
    "layernorm": N.OP_LAYERNORM,
    "rmsnorm": N.OP_RMSNORM,
    "softmax": N.OP_SOFTMAX,
    "rope": N.OP_ROPE,
    "elementwise": N.OP_ELEMENTWISE,
    "embedding": N.OP_EMBEDDING,
    "allreduce": N.OP_ALLREDUCE,
    "allgather": N.OP_ALLGATHER,
    "reducescatter": N.OP_REDUCESCATTER,
    "stream": N.OP_STREAM,
    "event_record": N.OP_EVENT_RECORD,
    "event_wait": N.OP_EVENT_WAIT,
    "reserve_sms": N.OP_RESERVE_SMS,
    "reduce_norm_gather": N.OP_REDUCE_NORM_GATHER,
    "gemm_rope": N.OP_GEMM_ROPE,
}


@dataclass
class ArgSpec:
    shape: tuple[int, ...]
    dtype: str
    name: str = ""


class Plan:
    """Entry name, argument signature, temporaries and operator list."""

    def __init__(self, entry: str, args: list[ArgSpec]):
        self.entry = entry
        self.args = list(args)
        self.temp_bytes: list[int] = []
        self.ops: list[PlanOp] = []

    # -- buffers ---------------------------------------------------------------------
    def arg(self, index: int) -> PView:
        a = self.args[index]
        return PView(index, tuple(a.shape), tuple(N.contiguous_strides(a.shape)), a.dtype)

    def temp(self, shape, dtype: str) -> PView:
        shape = tuple(int(d) for d in shape)
        self.temp_bytes.append(max(16, math.prod(shape) * dtype_bytes(dtype)))
        slot = len(self.args) + len(self.temp_bytes) - 1
        return PView(slot, shape, tuple(N.contiguous_strides(shape)), dtype)

    # -- operator emitters -------------------------------------------------------------
    def gemm(self, d, a, b, c=None, bias=None, residual=None, act="none", swiglu=False, force_simt=False):
        flags = (N.GEMM_ACCUMULATE_C if c is not None else 0) | (N.GEMM_SWIGLU if swiglu else 0) | (N.GEMM_FORCE_SIMT if force_simt else 0)
        self.ops.append(PlanOp("gemm", [d, a, b, c, bias, residual], {"act": act, "flags": flags}))
        return d

    def attention(self, o, q, k, v, scale: float, causal: bool = False):
        self.ops.append(PlanOp("attention", [o, q, k, v], {"scale": float(scale), "causal": bool(causal)}))
        return o

    def layernorm(self, out, x, gamma=None, beta=None, eps: float = 1e-5):
        self.ops.append(PlanOp("layernorm", [out, x, gamma, beta], {"eps": float(eps)}))
        return out

    def rmsnorm(self, out, x, weight=None, eps: float = 1e-5):
        self.ops.append(PlanOp("rmsnorm", [out, x, weight], {"eps": float(eps)}))
        return out

    def softmax(self, out, x):
        self.ops.append(PlanOp("softmax", [out, x]))
        return out

    def rope(self, x, theta: float = 10000.0, pos0: int = 0):
        self.ops.append(PlanOp("rope", [x], {"theta": float(theta), "pos0": int(pos0)}))
        return x

    def elementwise(self, kind: str, out, a=None, b=None, act="none", scalar: float = 0.0):
        self.ops.append(PlanOp("elementwise", [out, a, b], {"ew": kind, "act": act, "scalar": float(scalar)}))
        return out

    def embedding(self, out, ids, wte, wpe=None, period: int = 0):
        self.ops.append(PlanOp("embedding", [out, ids, wte, wpe], {"period": int(period)}))
        return out

    def allreduce(self, buf):
        """Sum over the tensor-parallel ranks, in place."""
        self.ops.append(PlanOp("allreduce", [buf]))
        return buf

    def reducescatter(self, out, inp):
        """``out`` = this rank's block of the sum over ranks of ``inp`` (world blocks)."""
        self.ops.append(PlanOp("reducescatter", [out, inp]))
        return out

    def gemm_rope(self, d, a, b, rope_cols: int, head_dim: int, seq: int, theta: float = 10000.0, pos0: int = 0):
        """``d = a @ b`` with the rotary embedding applied to its first ``rope_cols`` columns
        (heads of ``head_dim``; row r is position ``pos0 + r mod seq``)."""
        self.ops.append(PlanOp("gemm_rope", [d, a, b], {"rope_cols": int(rope_cols), "head_dim": int(head_dim), "seq": int(seq), "theta": float(theta), "pos0": int(pos0)}))
        return d

    def reduce_norm_gather(self, xn, part, h, weight, eps: float):
        """Fused reduce-scatter + residual add + RMSNorm + all-gather over symmetric memory:
        ``h += sum over ranks of part[my rows]`` (skipped when ``part`` is None), then
        ``xn[my rows]`` on every rank ``= rmsnorm(h) * weight``."""
        self.ops.append(PlanOp("reduce_norm_gather", [xn, part, h, weight], {"eps": float(eps)}))
        return xn

    # -- side stream: operators after ``stream(1)`` go to the context's second stream until
    # ``stream(0)``; numbered events order the two streams.
    def stream(self, side: int):
        self.ops.append(PlanOp("stream", [], {"index": int(side)}))

    def event_record(self, number: int):
        self.ops.append(PlanOp("event_record", [], {"index": int(number)}))

    def event_wait(self, number: int):
        self.ops.append(PlanOp("event_wait", [], {"index": int(number)}))

    def reserve_sms(self, n: int):
        """Persistent GEMMs leave ``n`` SMs to side-stream kernels from here on (0: none)."""
        self.ops.append(PlanOp("reserve_sms", [], {"index": int(n)}))

    def allgather(self, out, inp):
        self.ops.append(PlanOp("allgather", [out, inp]))
        return out

    # -- accounting ----------------------------------------------------------------------
    def total_flops(self) -> int:
        return sum(op.flops() for op in self.ops)

    def kinds(self) -> list[str]:
        """Operator kinds in launch order (the analogue of the ``kinds`` list the reference's
        nanoGPT builder keeps, examples/xegpu/nanoGPT_payload.py:58-75)."""
        return [op.kind if op.kind != "elementwise" else "ew:" + op.attrs["ew"] for op in self.ops]

    # -- native form -----------------------------------------------------------------------
    def to_native(self):
        nargs = len(self.args)
        sig = (N.ArgSig * max(nargs, 1))()
        for i, a in enumerate(self.args):
            sig[i].rank = len(a.shape)
            sig[i].dtype = N.DTYPE_FROM_NAME[a.dtype]
        temps = (ctypes.c_size_t * max(len(self.temp_bytes), 1))(*self.temp_bytes)
        ops = (N.Op * max(len(self.ops), 1))()
        for i, op in enumerate(self.ops):
            o = ops[i]
            o.kind = _KIND_CODES[op.kind]
            for j in range(N.LH_MAX_OPERANDS):
                o.operands[j].slot = -1
            for j, v in enumerate(op.operands):
                if v is not None:
                    o.operands[j] = v.to_native()
            at = op.attrs
            if op.kind == "gemm":
                o.i0, o.i1 = ACT_CODES[at.get("act", "none")], int(at.get("flags", 0)) | ((int(at.get("tile_n", 0)) // 8) << 8)
            elif op.kind == "attention":
                o.f0, o.i0 = at["scale"], int(at.get("causal", False))
            elif op.kind in ("layernorm", "rmsnorm", "reduce_norm_gather"):
                o.f0 = at.get("eps", 1e-5)
            elif op.kind == "rope":
                o.f0, o.i0 = at.get("theta", 10000.0), at.get("pos0", 0)
            elif op.kind == "elementwise":
                o.i0, o.i1, o.f0 = EW_CODES[at["ew"]], ACT_CODES[at.get("act", "none")], at.get("scalar", 0.0)
            elif op.kind == "embedding":
                o.i0 = at.get("period", 0)
            elif op.kind == "gemm_rope":
                o.i0, o.i1, o.i2, o.f0, o.f1 = at["rope_cols"], at["head_dim"], at["seq"], at["theta"], float(at["pos0"])
            elif op.kind in ("stream", "event_record", "event_wait", "reserve_sms"):
                o.i0 = at["index"]
        return sig, nargs, temps, len(self.temp_bytes), ops, len(self.ops)

    def __str__(self) -> str:
        lines = [f"plan @{self.entry}({', '.join('x'.join(map(str, a.shape)) + 'x' + a.dtype for a in self.args)})"]
        lines.append(f"  temps: {len(self.temp_bytes)} ({sum(self.temp_bytes)} bytes)")
        for op in self.ops:
            ops = ", ".join("-" if v is None else f"s{v.slot}{list(v.shape)}{v.dtype}" for v in op.operands)
            lines.append(f"  {op.kind}({ops}) {op.attrs}")
        return "\n".join(lines)
