"""Pipeline layer with the reference's names (lighthouse/pipeline/): descriptors, stages,
drivers and the target-based descriptor finder, for the CUDA dispatch target."""

from .descriptor import Descriptor, PipelineDescriptor
from .driver import BackendDriver, CompilerDriver, PipelineDriver, TransformDriver
from .finder import DESCRIPTORS_REPO, find_pipeline_file
from .helper import PipelineInterrupt
from .stage import CudaDispatchStage, Pass, PassStage, Stage, Transform, TransformStage

__all__ = [
    "BackendDriver", "CompilerDriver", "CudaDispatchStage", "DESCRIPTORS_REPO", "Descriptor", "Pass", "PassStage", "PipelineDescriptor",
    "PipelineDriver", "PipelineInterrupt", "Stage", "Transform", "TransformDriver", "TransformStage", "find_pipeline_file",
]
