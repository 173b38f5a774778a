"""Autoregressive generation helpers."""

from visionrl_b200.engine.ar.executor_base import (
    ARChunkResult, ARPipelineExecutorBase, align_pair, chunk_seed_offset,
    expand_prompt_major_prompts, max_peak_memory_mb, ordered_chunks, parse_ar_generation_spec,
    peak_memory_mb, require_rows, validate_chunk,
)
from visionrl_b200.engine.ar.sequence import ActiveSequence, ARSequenceKey
from visionrl_b200.engine.ar.spec import ARGenerationSpec
from visionrl_b200.engine.ar.token_scheduler import ARTokenBatch, ARTokenScheduler
from visionrl_b200.models.ar import ARStepResult

__all__ = [
    "ARChunkResult", "ARGenerationSpec", "ARPipelineExecutorBase", "ARSequenceKey", "ARStepResult", "ARTokenBatch",
    "ARTokenScheduler", "ActiveSequence", "align_pair", "chunk_seed_offset",
    "expand_prompt_major_prompts", "max_peak_memory_mb", "ordered_chunks",
    "parse_ar_generation_spec", "peak_memory_mb", "require_rows", "validate_chunk",
]
