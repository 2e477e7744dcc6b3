"""``PlanSession``: a plan instantiated on one GPU (native module + context), run with
device-resident torch tensors as arguments. This is what the decoder workloads and
``bench.py`` use; the ``Runner`` offers the same execution behind the reference's API."""

from __future__ import annotations

import ctypes
from ctypes import byref, c_double, c_void_p

import numpy as np

from .. import _native as N
from ..context import CudaContext, torch_dtype_code
from ..plan import Plan


class PlanSession:
    def __init__(self, plan: Plan, ctx: CudaContext | None = None, device: int = 0, use_graph: bool = False):
        self.plan = plan
        self._owns_ctx = ctx is None
        self.ctx = ctx if ctx is not None else CudaContext(device)
        sig, nargs, temps, ntemps, ops, nops = plan.to_native()
        handle = c_void_p()
        rc = self.ctx._lib.lh_b200_module_create(self.ctx.handle, plan.entry.encode(), sig, nargs, temps, ntemps, ops, nops, byref(handle))
        N.check(rc, self.ctx.handle, "lh_b200_module_create")
        self.handle = handle
        if use_graph:
            N.check(self.ctx._lib.lh_b200_module_use_graph(handle, 1), self.ctx.handle)

    def _pointers(self, args):
        if len(args) != len(self.plan.args):
            raise ValueError(f"plan '{self.plan.entry}' takes {len(self.plan.args)} arguments, got {len(args)}")
        ptrs = (c_void_p * max(len(args), 1))()
        for i, (t, spec) in enumerate(zip(args, self.plan.args)):
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"argument {i} ({spec.name}) must be a contiguous CUDA tensor")
            if tuple(t.shape) != tuple(spec.shape) or N.DTYPE_NAME[torch_dtype_code(t.dtype)] != spec.dtype:
                raise ValueError(f"argument {i} ({spec.name}) is {tuple(t.shape)} {t.dtype}, plan expects {spec.shape} {spec.dtype}")
            ptrs[i] = t.data_ptr()
        return ptrs

    def run(self, args, sync: bool = False) -> None:
        """Launches the plan's operators on the context's stream."""
        ptrs = self._pointers(args)
        N.check(self.ctx._lib.lh_b200_module_run(self.handle, ptrs, len(args)), self.ctx.handle, "lh_b200_module_run")
        if sync:
            self.ctx.sync()

    def benchmark(self, args, nruns: int = 20, nwarmup: int = 5, l2_flush_bytes: int = 0) -> np.ndarray:
        """Seconds per run, one CUDA-event pair per run on the context's stream."""
        ptrs = self._pointers(args)
        times = np.zeros((nruns,), dtype=np.float64)
        rc = self.ctx._lib.lh_b200_benchmark(self.handle, ptrs, len(args), times.ctypes.data_as(ctypes.POINTER(c_double)), nruns, nwarmup, l2_flush_bytes)
        N.check(rc, self.ctx.handle, "lh_b200_benchmark")
        return times

    def set_profiling(self, enable: bool = True) -> None:
        N.check(self.ctx._lib.lh_b200_module_set_profiling(self.handle, int(enable)), self.ctx.handle, "lh_b200_module_set_profiling")

    def op_times_ms(self) -> np.ndarray:
        """Per-operator durations (ms) of the last run made with profiling on."""
        n = len(self.plan.ops)
        ms = np.zeros((n,), dtype=np.float32)
        rc = self.ctx._lib.lh_b200_module_op_times(self.handle, ms.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), n)
        N.check(rc, self.ctx.handle, "lh_b200_module_op_times")
        return ms

    def timeline_ms(self) -> list[tuple[str, int, float, float]]:
        """(kind, stream, start, end) per operator of the last profiled run, in ms from the
        run's start; an operator's start is the end of the previous one on its stream (or its
        own end for the first), so waits show up as gaps inside the following operator."""
        n = len(self.plan.ops)
        ms = np.zeros((n,), dtype=np.float32)
        rc = self.ctx._lib.lh_b200_module_op_end_times(self.handle, ms.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), n)
        N.check(rc, self.ctx.handle, "lh_b200_module_op_end_times")
        out, stream, last = [], 0, {0: 0.0}
        for op, end in zip(self.plan.ops, ms):
            if op.kind == "stream":
                stream = op.attrs["index"]
                continue
            start = last.get(stream, float(end))
            out.append((op.kind, stream, float(start), float(end)))
            last[stream] = float(end)
        return out

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.ctx._lib.lh_b200_module_destroy(self.handle)
            self.handle = None
        if self._owns_ctx and self.ctx is not None:
            self.ctx.close()
        self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
