"""Model-free gathering of chunk payloads into an ``OutputBatch``
(reference: ``vrl/engine/gather.py:20-121``)."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any, Protocol

from visionrl_b200.engine.core.protocols import ChunkedFamilyPipelineExecutor, PipelineChunkResult
from visionrl_b200.engine.core.types import GenerationRequest, GenerationSampleSpec, OutputBatch


class ChunkGatherer(Protocol):
    def gather_chunks(self, request: GenerationRequest,
                      sample_specs: Sequence[GenerationSampleSpec],
                      chunks: Sequence[PipelineChunkResult]) -> OutputBatch: ...


def require_chunked_executor(executor: Any) -> ChunkedFamilyPipelineExecutor:
    if not callable(getattr(executor, "forward_chunk", None)) or not callable(
            getattr(executor, "gather_chunks", None)):
        raise TypeError(
            f"{type(executor).__name__} does not implement forward_chunk(...) and gather_chunks(...)"
        )
    return executor


def require_chunk_gatherer(gatherer: Any) -> ChunkGatherer:
    if not callable(getattr(gatherer, "gather_chunks", None)):
        raise TypeError(f"{type(gatherer).__name__} does not implement gather_chunks(...)")
    return gatherer


def gather_pipeline_chunks(gatherer: Any, request: GenerationRequest,
                           sample_specs: Sequence[GenerationSampleSpec],
                           chunks: Sequence[PipelineChunkResult]) -> OutputBatch:
    return require_chunk_gatherer(gatherer).gather_chunks(request, sample_specs, chunks)


def gather_diffusion_chunks(request: GenerationRequest,
                            sample_specs: Sequence[GenerationSampleSpec],
                            chunks: Sequence[PipelineChunkResult], *, model_family: str,
                            respect_cfg_flag: bool = True) -> OutputBatch:
    from visionrl_b200.engine.diffusion.denoise import build_diffusion_output_batch

    del model_family, respect_cfg_flag  # carried for compatibility; CFG is on iff guidance > 1
    return build_diffusion_output_batch(
        request=request, sample_specs=list(sample_specs), prompts=list(request.prompts),
        chunks=list(chunks), num_steps=int(request.sampling["num_steps"]),
    )


@dataclass(frozen=True, slots=True)
class DiffusionChunkGatherer:
    model_family: str
    respect_cfg_flag: bool = True

    def gather_chunks(self, request, sample_specs, chunks) -> OutputBatch:
        return gather_diffusion_chunks(request, sample_specs, chunks,
                                       model_family=self.model_family,
                                       respect_cfg_flag=self.respect_cfg_flag)


__all__ = [
    "ChunkGatherer", "DiffusionChunkGatherer", "gather_diffusion_chunks",
    "gather_pipeline_chunks", "require_chunk_gatherer", "require_chunked_executor",
]
