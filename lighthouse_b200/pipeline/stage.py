"""Pipeline stages. ``Stage.apply(module) -> module`` is the reference's contract
(lighthouse/pipeline/stage.py:105-116); the stages here act on ``PayloadModule`` objects.

* ``CudaDispatchStage`` — the routing hook of this backend: recognises the payload ops and
  attaches the plans the runner executes, in place of the CPU / XeGPU egress.
* ``PassStage`` — named passes. The names this backend defines are listed in ``PASSES``;
  upstream MLIR pass names that only prepare a module for LLVM lowering are accepted and do
  nothing (``NOOP_PASSES``) so that stage lists written for the reference still load; any
  other name is a ``ValueError``.
* ``TransformStage`` — a Python schedule file whose generator returns a ``Stage`` or a
  ``module -> module`` callable. Transform-dialect ``.mlir`` schedules need the MLIR
  bindings and are rejected with ``ValueError``.
"""

from __future__ import annotations

import importlib.util
import os
from abc import abstractmethod
from enum import Enum

from ..payload import lower as L
from ..payload import as_payload_module
from .descriptor import Descriptor, PipelineDescriptor


class Stage:
    @abstractmethod
    def apply(self, module):
        """Apply this stage to the module and return the transformed module."""


def _ensure_plans(module, fuse=False):
    if not module.plans:
        L.lower_module(module, fuse=fuse, fuse_attention_pattern=False)
    return module


def _pass_recognize(module, **_):
    module.plans.clear()
    return L.lower_module(module, fuse=False)


def _per_plan(fn):
    def run(module, **_):
        _ensure_plans(module)
        for plan in module.plans.values():
            fn(plan)
            L.compact_temps(plan)
        return module

    return run


PASSES = {
    "cuda-recognize": _pass_recognize,
    "cuda-fuse-epilogues": _per_plan(L.fuse_gemm_epilogues),
    "cuda-fuse-norm-cast": _per_plan(L.fuse_norm_cast),
    "cuda-fuse-attention": _per_plan(L.fuse_attention),
    "cuda-compact-temps": _per_plan(lambda plan: None),
}

# Upstream pass names that only matter on the way to LLVM IR; harmless to skip here.
NOOP_PASSES = {
    "canonicalize", "cse", "symbol-dce", "convert-linalg-to-loops", "fold-memref-alias-ops", "expand-strided-metadata", "lower-affine",
    "convert-vector-to-scf", "finalize-memref-to-llvm", "convert-scf-to-cf", "convert-vector-to-llvm", "convert-math-to-llvm",
    "convert-math-to-libm", "convert-to-llvm", "reconcile-unrealized-casts", "one-shot-bufferize", "convert-func-to-llvm",
}


class Pass:
    """Name + options of a pass, from a ``Descriptor``."""

    def __init__(self, desc: Descriptor):
        if not isinstance(desc, Descriptor):
            raise ValueError(f"Pass must be initialized with a Descriptor, got {type(desc)}")
        self.name = desc.basename
        self.options = desc.opts

    def __str__(self) -> str:
        if not self.options:
            return self.name
        return f"{self.name}{{{' '.join(f'{k}={v}' for k, v in self.options.items())}}}"


class PassStage(Stage):
    def __init__(self, passes: list[Pass], context=None):
        self.context = context
        self.passes = passes
        for p in passes:
            if p.name not in PASSES and p.name not in NOOP_PASSES:
                raise ValueError(f"Unknown pass '{p.name}' for the CUDA backend (known: {sorted(PASSES)})")

    def apply(self, module):
        if module is None:
            raise ValueError("Missing module to apply passes to.")
        for p in self.passes:
            if p.name in PASSES:
                module = PASSES[p.name](module, **p.options)
        return module

    def __str__(self) -> str:
        return f"PassStage({[str(p) for p in self.passes]})"


class Transform:
    """A schedule file: ``.py`` with ``[gen=function]`` and ``{options}``."""

    class Type(Enum):
        MLIR = 1
        Python = 2

    def __init__(self, desc: Descriptor):
        if not isinstance(desc, Descriptor):
            raise ValueError(f"Transform must be initialized with a Descriptor, got {type(desc)}")
        if desc.basename.endswith(".mlir"):
            self.type = Transform.Type.MLIR
        elif desc.basename.endswith(".py"):
            self.type = Transform.Type.Python
        else:
            raise ValueError(f"Unsupported transform file type: {desc.basename}")
        self.filename = desc.basename
        self.options = desc.opts
        self.generator = desc.args.get("gen", "create_schedule")
        self.sequence = desc.args.get("seq", "")

    def __str__(self) -> str:
        return self.filename if not self.options else f"{self.filename}{{{self.options}}}"


def import_python_module(path: str):
    if path is None or not os.path.exists(path):
        raise ValueError(f"Path to the module does not exist: {path}")
    spec = importlib.util.spec_from_file_location("lh_b200_schedule_" + os.path.splitext(os.path.basename(path))[0], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class TransformStage(Stage):
    def __init__(self, transform, context=None):
        self.context = context
        if isinstance(transform, Stage) or callable(getattr(transform, "apply", None)):
            self.inner, self.label = transform, str(transform)
            return
        if not isinstance(transform, Transform):
            raise ValueError(f"Unsupported transform: {type(transform)}")
        if transform.type == Transform.Type.MLIR:
            raise ValueError(f"Transform-dialect schedule {transform.filename} needs the MLIR bindings; the CUDA backend takes Python schedules and 'backend:' stages")
        mod = import_python_module(transform.filename)
        if not hasattr(mod, transform.generator):
            raise ValueError(f"Transform module '{transform.filename}' does not define a '{transform.generator}' generator function.")
        self.inner = getattr(mod, transform.generator)(**transform.options)
        self.label = str(transform)
        if not (callable(self.inner) or callable(getattr(self.inner, "apply", None))):
            raise ValueError(f"Generator '{transform.generator}' of {transform.filename} must return a Stage or a callable")

    def apply(self, module):
        if module is None:
            raise ValueError("Missing module to apply transformations to.")
        out = self.inner.apply(module) if hasattr(self.inner, "apply") else self.inner(module)
        return module if out is None else out

    def __str__(self) -> str:
        return f"TransformStage({self.label})"


class CudaDispatchStage(Stage):
    """Recognise + fuse + attach plans. Options: ``fuse`` (GEMM epilogues and norm+cast),
    ``fuse_attention`` (flash-attention rewrite)."""

    def __init__(self, fuse: bool = True, fuse_attention: bool = True, **unknown):
        if unknown:
            raise ValueError(f"Unknown options for the cuda backend stage: {sorted(unknown)}")
        self.fuse, self.fuse_attention = bool(fuse), bool(fuse_attention)

    def apply(self, module):
        module = as_payload_module(module, lower=False)
        module.plans.clear()
        return L.lower_module(module, fuse=self.fuse, fuse_attention_pattern=self.fuse_attention)

    def __str__(self) -> str:
        return f"CudaDispatchStage(fuse={self.fuse}, fuse_attention={self.fuse_attention})"


BACKENDS = {"cuda": CudaDispatchStage}
