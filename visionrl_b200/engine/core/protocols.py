"""Executor protocols (reference: ``vrl/engine/core/protocols.py:18-67``)."""

from __future__ import annotations

from collections.abc import Sequence
from typing import TYPE_CHECKING, Protocol, runtime_checkable

if TYPE_CHECKING:
    from visionrl_b200.engine.core.types import (
        GenerationRequest, GenerationSampleSpec, OutputBatch, WorkloadSignature,
    )
    from visionrl_b200.engine.microbatching import MicroBatchPlan


class PipelineChunkResult(Protocol):
    """Family-specific payload of one micro-batch, before gathering."""


@runtime_checkable
class FamilyPipelineExecutor(Protocol):
    family: str
    task: str

    def workload_signature(self, request: "GenerationRequest") -> "WorkloadSignature": ...

    def forward(self, request: "GenerationRequest",
                sample_specs: "list[GenerationSampleSpec]") -> "OutputBatch": ...


@runtime_checkable
class BatchedFamilyPipelineExecutor(FamilyPipelineExecutor, Protocol):
    def forward_batch(
        self, requests: "list[GenerationRequest]",
        sample_specs_by_request: "dict[str, list[GenerationSampleSpec]]",
    ) -> "dict[str, OutputBatch]": ...


@runtime_checkable
class ChunkedFamilyPipelineExecutor(FamilyPipelineExecutor, Protocol):
    def forward_chunk(self, request: "GenerationRequest",
                      chunk: "MicroBatchPlan") -> PipelineChunkResult: ...

    def gather_chunks(
        self, request: "GenerationRequest", sample_specs: "Sequence[GenerationSampleSpec]",
        chunks: "Sequence[PipelineChunkResult]",
    ) -> "OutputBatch": ...
