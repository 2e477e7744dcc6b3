"""Pipeline helpers (the part of lighthouse/pipeline/helper.py that does not need MLIR)."""


class PipelineInterrupt(Exception):
    """Signals early termination of a pipeline (e.g. to dump the module at a stage)."""
