"""``Runner`` for the CUDA backend: same constructor and methods as the reference's
``lighthouse.execution.runner.Runner`` (lighthouse/execution/runner.py:42-330), with the
MLIR ExecutionEngine replaced by the native sm_100a library.

    runner = Runner(module, mem_manager_cls=GPUMemoryManager)
    runner.execute("payload", host_buffers, argument_access_callback=cb)
    times = runner.benchmark(host_buffers, nruns=100, nwarmup=10)   # seconds per run

``module`` is a payload the CUDA dispatch stage has recognised (or can recognise):
a ``PayloadModule``, MLIR text, a path to an ``.mlir`` file, an object whose ``str()`` is
MLIR text (an ``ir.Module`` when the MLIR bindings exist), or a ``Plan``.
"""

from __future__ import annotations

import ctypes
import os
import typing
from collections.abc import Callable
from contextlib import contextmanager
from ctypes import byref, c_double, c_void_p
from functools import partial

import numpy as np

from .. import _native as N
from ..context import CudaContext
from ..plan import Plan
from ..utils.memref import make_descriptor, to_packed_args
from .memory_manager import CudaMemoryManager, ExternalMemoryManager, MemoryManager
from .target import TargetInfo


class RunnerCallable(typing.Protocol):
    """``argument_access_callback(inputs, execution_engine=..., memory_manager=...)``."""

    def __call__(self, inputs: list[ctypes.Structure], execution_engine, memory_manager: MemoryManager | None) -> None: ...


class BenchWrapperSchedule:
    """What ``Runner.get_bench_wrapper_schedule`` returns: a pipeline stage that marks which
    function ``benchmark()`` times. The reference wraps the function in a ``__benchmark``
    function at IR level (wrap_in_benching_func.py:29-65); here timing is done by
    ``lh_b200_benchmark`` with CUDA events, so the stage only records the name."""

    def __init__(self, payload_func: str):
        self.payload_func = payload_func

    def apply(self, module):
        module.bench_target = self.payload_func
        return module

    def __str__(self) -> str:
        return f"BenchWrapperSchedule({self.payload_func})"


class Runner:
    """Executes and benchmarks recognised payload modules on a B200."""

    payload_benchmark_function_name: str = "__benchmark"

    def __init__(
        self,
        module,
        mem_manager_cls: type | None = None,
        shared_libs: list[str] | None = None,
        opt_level: int = 3,
        target: TargetInfo = None,
        device: int | None = None,
        context: CudaContext | None = None,
    ):
        from ..payload import as_payload_module  # late import: payload imports nothing from execution

        self.target = target if target else TargetInfo.cuda()
        self.mem_manager_cls = mem_manager_cls
        self.shared_libs = list(shared_libs) if shared_libs else []  # accepted for signature parity; unused
        self.opt_level = opt_level
        if device is None:
            device = int(os.environ.get("LOCAL_RANK", "0"))
        self._owns_engine = context is None
        self.engine = context if context is not None else CudaContext(device)
        self.payload = as_payload_module(module)
        self._modules: dict[str, c_void_p] = {}
        self.use_graph = False

    # -- native modules ------------------------------------------------------------------
    def _plan(self, name: str) -> Plan:
        plans = self.payload.plans
        if name not in plans:
            raise ValueError(f"payload has no function '{name}' (has: {sorted(plans)})")
        return plans[name]

    def _native_module(self, name: str) -> c_void_p:
        if name in self._modules:
            return self._modules[name]
        plan = self._plan(name)
        sig, nargs, temps, ntemps, ops, nops = plan.to_native()
        handle = c_void_p()
        rc = self.engine._lib.lh_b200_module_create(self.engine.handle, name.encode(), sig, nargs, temps, ntemps, ops, nops, byref(handle))
        N.check(rc, self.engine.handle, "lh_b200_module_create")
        if self.use_graph:
            self.engine._lib.lh_b200_module_use_graph(handle, 1)
        self._modules[name] = handle
        return handle

    def close(self) -> None:
        for h in self._modules.values():
            self.engine._lib.lh_b200_module_destroy(h)
        self._modules.clear()
        if self._owns_engine and self.engine is not None:
            self.engine.close()
        self.engine = None

    def __del__(self):
        try:
            if self.engine is not None:
                self.close()
        except Exception:
            pass

    # -- argument handling ------------------------------------------------------------------
    @contextmanager
    def _host_clone_manager(self, plan: Plan, inputs: list[np.ndarray]):
        """No memory manager given: the reference runs in place on the host arrays
        (runner.py:139-144). This backend has no CPU path, so the arrays are cloned to the
        device and every argument the payload writes is copied back in place afterwards."""
        mm = CudaMemoryManager(self.engine)
        written = {op.operands[0].slot for op in plan.ops if op.operands and op.operands[0] is not None}
        written |= {op.operands[0].slot for op in plan.ops if op.kind == "rope"}
        with mm.clone_host_buffers(inputs) as bufs:
            yield bufs
            for i, (host, buf) in enumerate(zip(inputs, bufs)):
                if i in written:
                    mm.copy(buf, host)

    def _check_args(self, plan: Plan, arrays) -> None:
        if len(arrays) != len(plan.args):
            raise ValueError(f"function '{plan.entry}' takes {len(plan.args)} arguments, got {len(arrays)}")
        for i, (spec, a) in enumerate(zip(plan.args, arrays)):
            if tuple(a.shape) != tuple(spec.shape):
                raise ValueError(f"argument {i} has shape {tuple(a.shape)}, payload expects {tuple(spec.shape)}")

    def _execute_kernel(
        self,
        host_input_buffers: list,
        payload_function_name: str = "",
        argument_access_callback: Callable | None = None,
        nruns: int = 100,
        nwarmup: int = 10,
        benchmark: bool = True,
    ) -> np.ndarray | None:
        if host_input_buffers is None:
            raise ValueError("host_input_buffers must be provided")
        if benchmark:
            name = getattr(self.payload, "bench_target", None)
            if name is None:
                if len(self.payload.plans) != 1:
                    raise ValueError("benchmark needs the bench wrapper stage (Runner.get_bench_wrapper_schedule) to name the function")
                name = next(iter(self.payload.plans))
        else:
            name = payload_function_name
        plan = self._plan(name)
        self._check_args(plan, host_input_buffers)

        if self.mem_manager_cls is None:
            if any(not isinstance(buf, np.ndarray) for buf in host_input_buffers):
                raise ValueError("host_input_buffers must be numpy arrays when no mem_manager_cls is provided")
            mem_manager = None
            allocator = partial(self._host_clone_manager, plan, host_input_buffers)
        elif issubclass(self.mem_manager_cls, ExternalMemoryManager):
            mem_manager = self.mem_manager_cls(self.engine)
            allocator = partial(mem_manager.get_memrefs, host_input_buffers)
        elif issubclass(self.mem_manager_cls, CudaMemoryManager):
            mem_manager = self.mem_manager_cls(self.engine)
            allocator = partial(mem_manager.clone_host_buffers, host_input_buffers)
        else:
            raise ValueError(f"Unsupported mem_manager_cls type: {self.mem_manager_cls}")

        module = self._native_module(name)
        lib = self.engine._lib
        with allocator() as inputs:
            if benchmark:
                time_array = np.zeros((nruns,), dtype=np.float64)
                ptrs = (c_void_p * max(len(inputs), 1))(*[_data_ptr(d, spec.dtype) for d, spec in zip(inputs, plan.args)])
                rc = lib.lh_b200_benchmark(module, ptrs, len(inputs), time_array.ctypes.data_as(ctypes.POINTER(c_double)), nruns, nwarmup, 0)
                N.check(rc, self.engine.handle, "lh_b200_benchmark")
            else:
                time_array = None
                args = to_packed_args(inputs)
                rc = lib.lh_b200_invoke(module, name.encode(), args, len(inputs))
                N.check(rc, self.engine.handle, "lh_b200_invoke")
                self.engine.sync()
            if argument_access_callback is not None:
                argument_access_callback(inputs, execution_engine=self.engine, memory_manager=mem_manager)
        return time_array

    def benchmark(self, host_input_buffers: list, argument_access_callback: RunnerCallable = None, nruns: int = 100, nwarmup: int = 10) -> np.ndarray:
        """Times the payload: ``nwarmup`` untimed runs, then ``nruns`` runs timed one by one
        with CUDA events; returns seconds per run (runner.py:226-242 contract)."""
        return self._execute_kernel(host_input_buffers=host_input_buffers, argument_access_callback=argument_access_callback, nruns=nruns, nwarmup=nwarmup, benchmark=True)

    def execute(self, payload_function_name: str, host_input_buffers: list, argument_access_callback: RunnerCallable = None) -> None:
        """Runs the named function; results are written in place into the argument buffers."""
        self._execute_kernel(host_input_buffers=host_input_buffers, payload_function_name=payload_function_name, argument_access_callback=argument_access_callback, benchmark=False)

    def dump_object_file(self, file_name: str) -> str:
        """The reference dumps the JIT's object file; the analogue here is the plan listing."""
        if not file_name:
            raise ValueError("non-empty file_name must be provided")
        with open(file_name, "w") as f:
            for plan in self.payload.plans.values():
                f.write(str(plan) + "\n")
        return file_name

    @staticmethod
    def get_bench_wrapper_schedule(payload_func: str) -> BenchWrapperSchedule:
        return BenchWrapperSchedule(payload_func)

    @staticmethod
    def get_gpu_argument_access_callback(host_buffer: np.ndarray, arg_index: int = 0) -> RunnerCallable:
        """Returns a callback that copies device-allocated function argument to the host."""

        def argument_access_callback(inputs, *, memory_manager, **kwargs):
            memory_manager.copy(inputs[arg_index], host_buffer)

        return argument_access_callback

    @staticmethod
    def make_function_callable(module, func_name: str) -> None:
        """The reference sets ``llvm.emit_c_interface`` on the function; every recognised
        function is callable here, so this only checks that the function exists."""
        from ..payload import as_payload_module

        pm = as_payload_module(module, lower=False)
        if func_name not in pm.funcs:
            raise ValueError(f"payload has no function '{func_name}'")


def _data_ptr(desc, dtype: str) -> int:
    return (desc.aligned or 0) + desc.offset * N.DTYPE_SIZE[N.DTYPE_FROM_NAME[dtype]]


CudaRunner = Runner
