"""Engine core: payload types, executor protocols, registry, worker and runtime."""
from visionrl_b200.engine.core.protocols import (
    BatchedFamilyPipelineExecutor, ChunkedFamilyPipelineExecutor, FamilyPipelineExecutor, PipelineChunkResult,
)
from visionrl_b200.engine.core.registry import ExecutorKey, FamilyPipelineRegistry
from visionrl_b200.engine.core.runtime import GenerationRuntime, RolloutBackend
from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec
from visionrl_b200.engine.core.types import (
    GenerationMetrics, GenerationRequest, GenerationSampleSpec, OutputBatch, RolloutDebugTensors,
    RolloutDenoisingEnv, RolloutDitTrajectory, RolloutTrajectoryData, WorkloadSignature,
)
from visionrl_b200.engine.core.worker import GenerationIdFactory, GenerationWorker

__all__ = [
    "BatchedFamilyPipelineExecutor", "ChunkedFamilyPipelineExecutor", "ExecutorKey", "FamilyPipelineExecutor",
    "FamilyPipelineRegistry", "GenerationIdFactory", "GenerationMetrics", "GenerationRequest", "GenerationRuntime",
    "GenerationRuntimeSpec", "GenerationSampleSpec", "GenerationWorker", "OutputBatch", "PipelineChunkResult",
    "RolloutBackend", "RolloutDebugTensors", "RolloutDenoisingEnv", "RolloutDitTrajectory", "RolloutTrajectoryData",
    "WorkloadSignature",
]
