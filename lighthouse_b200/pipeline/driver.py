"""Pipeline drivers with the reference's classes and methods
(lighthouse/pipeline/driver.py:12-235): ``PipelineDriver`` (a list of stages applied in
order), ``TransformDriver``, ``BackendDriver`` and ``CompilerDriver`` (file in, module out).
The ``context`` argument the reference threads through (an ``ir.Context``) is accepted and
ignored: payloads here are plain Python objects."""

from __future__ import annotations

import os

from ..payload import as_payload_module
from ..payload.ir import PayloadModule
from . import stage as lhs
from .descriptor import Descriptor, PipelineDescriptor


class PipelineDriver:
    def __init__(self, context=None):
        self.context = context
        self.stages: list[lhs.Stage] = []

    def add_pass(self, stage: Descriptor) -> None:
        self.stages.append(lhs.PassStage([lhs.Pass(stage)], self.context))

    def add_transform(self, stage) -> None:
        if isinstance(stage, Descriptor):
            self.stages.append(lhs.TransformStage(lhs.Transform(stage), self.context))
        elif isinstance(stage, lhs.Stage) or callable(getattr(stage, "apply", None)):
            self.stages.append(lhs.TransformStage(stage, self.context))
        else:
            raise ValueError(f"Unsupported stage type: {type(stage)}")

    def add_backend(self, stage: Descriptor) -> None:
        if stage.basename not in lhs.BACKENDS:
            raise ValueError(f"Unknown backend '{stage.basename}' (known: {sorted(lhs.BACKENDS)})")
        self.stages.append(lhs.BACKENDS[stage.basename](**stage.opts))

    def add_stage(self, stage) -> None:
        """A ready stage, anything with ``apply(module)``, or a descriptor - which may name a
        backend, a transform file, a pipeline YAML (expanded into its stages) or a pass."""
        if isinstance(stage, lhs.Stage):
            self.stages.append(stage)
        elif not isinstance(stage, Descriptor):
            if not callable(getattr(stage, "apply", None)):
                raise ValueError(f"Unsupported stage type: {type(stage)}")
            self.stages.append(lhs.TransformStage(stage, self.context))
        elif stage.is_backend():
            self.add_backend(stage)
        elif not os.path.exists(stage.basename):
            self.add_pass(stage)
        else:
            extension = os.path.splitext(stage.basename)[1]
            if extension in (".mlir", ".py"):
                self.add_transform(stage)
            elif extension == ".yaml":
                self.add_stages(PipelineDescriptor(stage).get_stages())
            else:
                raise ValueError(f"Unknown file type '{extension}' for stage '{stage}'.")

    def add_stages(self, stages: list) -> None:
        for s in stages:
            self.add_stage(s)

    def add_descriptor(self, stage: Descriptor) -> None:
        for s in PipelineDescriptor(stage).get_stages():
            self.add_stage(s)

    def apply(self, module, print_after_all: bool = False):
        for stage in self.stages:
            module = stage.apply(module)
            if print_after_all:
                print(f"After stage {stage}:\n{module}")
                for plan in getattr(module, "plans", {}).values():
                    print(plan)
        return module

    def __len__(self):
        return len(self.stages)

    def reset(self):
        self.stages = []


class TransformDriver(PipelineDriver):
    """Runs a sequence of schedules (stages or ``module -> module`` callables)."""

    def __init__(self, schedules: list):
        if not isinstance(schedules, list) or not schedules:
            raise ValueError("Schedules must be a non-empty list")
        super().__init__(None)
        for s in schedules:
            self.add_stage(s)


class BackendDriver(PipelineDriver):
    """Prepares a module for execution: checks the entry point, optionally marks it as the
    benchmark target. ``result_to_args`` (results moved to leading arguments,
    convert_func_results_to_args.py:14-55 in the reference) is not needed: payloads for this
    backend already take their results as arguments, and one that does not is rejected at
    recognition."""

    def __init__(self, module, entry_point: str, result_to_args: bool = False, benchmark: bool = False):
        from ..execution.runner import Runner

        if not isinstance(module, PayloadModule):
            raise ValueError("Module must be a PayloadModule")
        if not entry_point:
            raise ValueError("Entry point must be a valid function name")
        super().__init__(None)
        Runner.make_function_callable(module, entry_point)
        if benchmark:
            self.add_stage(Runner.get_bench_wrapper_schedule(entry_point))


class CompilerDriver:
    """File in, recognised module out. The pipeline is fixed after the first ``run``;
    ``reset`` clears it."""

    def __init__(self, filename: str, stages: list[str] = []):
        self.context = None
        self.module = None
        if filename:
            self.import_payload(filename)
        self.pipeline = PipelineDriver(self.context)
        self.pipeline_fixed = False
        if stages:
            self.add_stages(list(stages))

    def import_payload(self, path: str) -> None:
        if self.module is not None:
            raise ValueError("Module already imported. Reset to start again.")
        if path is None:
            raise ValueError("Path to the module must be provided.")
        if not os.path.exists(path):
            raise ValueError(f"Path to the module does not exist: {path}")
        self.module = as_payload_module(path, lower=False)

    def _check_open(self) -> None:
        if self.pipeline_fixed:
            raise ValueError("Pipeline is fixed. Reset to start again.")

    def add_stage(self, stage) -> None:
        self._check_open()
        self.pipeline.add_stage(Descriptor(stage) if isinstance(stage, str) else stage)

    def add_stages(self, stages: list) -> None:
        self._check_open()
        for s in stages:
            self.pipeline.add_stage(Descriptor(s) if isinstance(s, str) else s)

    def add_module_stage(self, stage_module) -> None:
        self._check_open()
        self.pipeline.add_stage(stage_module)

    def reset(self) -> None:
        self.pipeline.reset()
        self.module = None
        self.pipeline_fixed = False

    def run(self, print_after_all: bool = False):
        if self.module is None:
            raise ValueError("Module must not be empty.")
        if len(self.pipeline) == 0:
            raise ValueError("Pipeline must have at least one stage.")
        module = self.pipeline.apply(self.module, print_after_all=print_after_all)
        self.pipeline_fixed = True
        self.module = None
        return module
