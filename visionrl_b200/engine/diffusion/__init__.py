"""Diffusion generation: denoise loop, executor base and parsed specs."""

from visionrl_b200.engine.diffusion.denoise import (
    DiffusionChunkResult, DiffusionDenoiseConfig, build_diffusion_output_batch, peak_memory_mb,
    repeat_tensor_batch, run_diffusion_denoise_chunk, select_sde_window,
)
from visionrl_b200.engine.diffusion.executor_base import DiffusionPipelineExecutorBase
from visionrl_b200.engine.diffusion.spec import (
    BaseDiffusionGenerationSpec, DiffusionGenerationSpec, SDEDiffusionSpec,
)

__all__ = [
    "BaseDiffusionGenerationSpec", "DiffusionChunkResult", "DiffusionDenoiseConfig",
    "DiffusionGenerationSpec", "DiffusionPipelineExecutorBase", "SDEDiffusionSpec",
    "build_diffusion_output_batch", "peak_memory_mb", "repeat_tensor_batch",
    "run_diffusion_denoise_chunk", "select_sde_window",
]
