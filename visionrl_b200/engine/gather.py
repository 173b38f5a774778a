"""Assembling the chunks one consumer ran into one ``OutputBatch``.

In the one-process-per-GPU runtime every rank runs only ITS chunks of a request and gathers only
those: the tensors of a chunk never leave the GPU that produced them, so "gathering" here is a
device-side concatenation plus bookkeeping, never a transfer.  A gatherer is therefore a small
model-free object (it can be built from an import path on any rank, before any weights exist)
whose one duty is to turn ``(request, sample specs, chunk results)`` into an ``OutputBatch`` and
to refuse input that does not add up — chunk results that cover more or fewer samples than the
specs name would silently misalign rewards and trajectories further down.

Behavioural reference: ``vrl/engine/gather.py:20-121`` (there the chunks arrive as CPU tensors
from Ray actors and are concatenated on the driver).
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any, Protocol, runtime_checkable

from visionrl_b200.engine.core.protocols import ChunkedFamilyPipelineExecutor, PipelineChunkResult
from visionrl_b200.engine.core.types import GenerationRequest, GenerationSampleSpec, OutputBatch


@runtime_checkable
class ChunkGatherer(Protocol):
    def gather_chunks(self, request: GenerationRequest,
                      sample_specs: Sequence[GenerationSampleSpec],
                      chunks: Sequence[PipelineChunkResult]) -> OutputBatch: ...


def _missing(obj: Any, names: tuple[str, ...]) -> list[str]:
    return [n for n in names if not callable(getattr(obj, n, None))]


def require_chunked_executor(executor: Any) -> ChunkedFamilyPipelineExecutor:
    """``executor`` unchanged, or ``TypeError`` naming what it lacks to run single chunks."""
    if _missing(executor, ("forward_chunk", "gather_chunks")):
        raise TypeError(f"{type(executor).__name__} does not implement forward_chunk(...) and "
                        "gather_chunks(...)")
    return executor


def require_chunk_gatherer(gatherer: Any) -> ChunkGatherer:
    if _missing(gatherer, ("gather_chunks",)):
        raise TypeError(f"{type(gatherer).__name__} does not implement gather_chunks(...)")
    return gatherer


def chunk_rows(chunk: Any) -> int | None:
    """Samples a chunk result holds, when it can tell (leading dimension of its log-probs)."""
    for name in ("log_probs", "token_log_probs"):
        shape = getattr(getattr(chunk, name, None), "shape", None)
        if shape is not None and len(shape) > 0:
            return int(shape[0])
    count = getattr(chunk, "sample_count", None)
    return int(count) if count else None


def check_coverage(sample_specs: Sequence[GenerationSampleSpec], chunks: Sequence[Any]) -> None:
    """The chunks together hold exactly one row per sample spec (when they can be counted)."""
    rows = [chunk_rows(c) for c in chunks]
    if rows and all(r is not None for r in rows) and sum(rows) != len(sample_specs):
        raise ValueError(f"chunk results hold {sum(rows)} samples but {len(sample_specs)} sample "
                         "specs were given; they would be misaligned")


def gather_pipeline_chunks(gatherer: Any, request: GenerationRequest,
                           sample_specs: Sequence[GenerationSampleSpec],
                           chunks: Sequence[PipelineChunkResult]) -> OutputBatch:
    return require_chunk_gatherer(gatherer).gather_chunks(request, sample_specs, chunks)


def gather_diffusion_chunks(request: GenerationRequest,
                            sample_specs: Sequence[GenerationSampleSpec],
                            chunks: Sequence[PipelineChunkResult], *, model_family: str,
                            respect_cfg_flag: bool = True) -> OutputBatch:
    """Diffusion chunks → one batch.  ``model_family`` and ``respect_cfg_flag`` belong to the
    call signature families and registries use; classifier-free guidance is decided by
    ``guidance_scale > 1`` alone, so neither changes the result."""
    from visionrl_b200.engine.diffusion.denoise import build_diffusion_output_batch

    del model_family, respect_cfg_flag
    specs, parts = list(sample_specs), list(chunks)
    check_coverage(specs, parts)
    return build_diffusion_output_batch(request=request, sample_specs=specs,
                                        prompts=list(request.prompts), chunks=parts,
                                        num_steps=int(request.sampling["num_steps"]))


@dataclass(frozen=True, slots=True)
class DiffusionChunkGatherer:
    """Stateless, picklable gatherer of the diffusion families (named by import path in the
    family registry)."""

    model_family: str
    respect_cfg_flag: bool = True

    def gather_chunks(self, request, sample_specs, chunks) -> OutputBatch:
        return gather_diffusion_chunks(request, sample_specs, chunks,
                                       model_family=self.model_family,
                                       respect_cfg_flag=self.respect_cfg_flag)


__all__ = [
    "ChunkGatherer", "DiffusionChunkGatherer", "check_coverage", "chunk_rows",
    "gather_diffusion_chunks", "gather_pipeline_chunks", "require_chunk_gatherer",
    "require_chunked_executor",
]
