"""Helpers shared by autoregressive family executors: spec parsing, prompt-major
expansion, chunk validation/ordering, seed offsets and cond/uncond padding
(reference: ``vrl/engine/ar/executor_base.py:37-294``)."""

from __future__ import annotations

from collections.abc import Sequence
from typing import Any, Protocol, TypeVar

import torch

from visionrl_b200.engine.ar.spec import ARGenerationSpec
from visionrl_b200.engine.batching import forward_batch_by_merging_prompts
from visionrl_b200.engine.core.types import GenerationRequest, GenerationSampleSpec, OutputBatch
from visionrl_b200.engine.diffusion.denoise import peak_memory_mb
from visionrl_b200.engine.microbatching import MicroBatchPlan


class ARChunkResult(Protocol):
    prompt_index: int
    sample_start: int
    sample_count: int
    peak_memory_mb: float | None


TChunk = TypeVar("TChunk", bound=ARChunkResult)


def _int_field(sampling: dict[str, Any], key: str, default: int | None) -> int:
    if key in sampling:
        return int(sampling[key])
    if default is None:
        raise KeyError(key)
    return int(default)


def parse_ar_generation_spec(request: GenerationRequest, *, default_image_token_num=576,
                             default_image_size=384, default_max_text_length=256) -> ARGenerationSpec:
    s = request.sampling
    seed = s.get("seed")
    return ARGenerationSpec(
        image_token_num=_int_field(s, "image_token_num", default_image_token_num),
        image_size=_int_field(s, "image_size", default_image_size),
        max_text_length=_int_field(s, "max_text_length", default_max_text_length),
        seed=None if seed is None else int(seed),
        use_ar_scheduler=bool(s.get("use_ar_scheduler", False)),
    )


def expand_prompt_major_prompts(request: GenerationRequest) -> list[str]:
    return [p for p in request.prompts for _ in range(int(request.samples_per_prompt))]


def _check_range(request: GenerationRequest, prompt_index: int, start: int, count: int) -> None:
    if not 0 <= prompt_index < len(request.prompts):
        raise ValueError(f"chunk.prompt_index={prompt_index} is out of range")
    if start < 0 or count < 1:
        raise ValueError("chunk sample range must have non-negative start and positive count")
    if start + count > request.samples_per_prompt:
        raise ValueError(
            "chunk sample range exceeds request.samples_per_prompt: "
            f"{start}:{start + count} > {request.samples_per_prompt}"
        )


def validate_chunk(request: GenerationRequest, chunk: MicroBatchPlan) -> None:
    _check_range(request, chunk.prompt_index, chunk.sample_start, chunk.sample_count)
    if chunk.prompt != request.prompts[chunk.prompt_index]:
        raise ValueError("chunk.prompt does not match request.prompts[chunk.prompt_index]")


def require_rows(name: str, value: Any, count: int) -> None:
    shape = getattr(value, "shape", None)
    if shape is None or len(shape) < 1:
        raise ValueError(f"chunk {name} must have a leading batch dimension")
    if int(shape[0]) != count:
        raise ValueError(f"chunk {name} has {shape[0]} rows, expected {count}")


def ordered_chunks(request: GenerationRequest, sample_specs: Sequence[GenerationSampleSpec],
                   chunks: Sequence[TChunk], *, row_fields: Sequence[str] = ()) -> list[TChunk]:
    if not chunks:
        raise ValueError("chunks must be non-empty")
    ordered = sorted(chunks, key=lambda c: (int(c.prompt_index), int(c.sample_start)))
    covered: list[tuple[int, int]] = []
    for c in ordered:
        p, start, count = int(c.prompt_index), int(c.sample_start), int(c.sample_count)
        _check_range(request, p, start, count)
        for name in row_fields:
            require_rows(name, getattr(c, name), count)
        covered.extend((p, j) for j in range(start, start + count))
    if covered != [(s.prompt_index, s.sample_index) for s in sample_specs]:
        raise ValueError("AR chunks do not cover sample_specs in prompt-major sample order")
    return ordered


def chunk_seed_offset(request: GenerationRequest, chunk: MicroBatchPlan) -> int:
    return chunk.prompt_index * int(request.samples_per_prompt) + chunk.sample_start


def max_peak_memory_mb(chunks: Sequence[ARChunkResult]) -> float | None:
    peaks = [c.peak_memory_mb for c in chunks if c.peak_memory_mb is not None]
    return max(peaks) if peaks else None


def align_pair(a_ids, a_mask, b_ids, b_mask, pad_id: int = 0):
    """Right-pad two ``[B, L]`` id/mask pairs to the longer length."""
    width = max(a_ids.shape[1], b_ids.shape[1])

    def pad(ids, mask):
        extra = width - ids.shape[1]
        if extra == 0:
            return ids, mask
        return (torch.nn.functional.pad(ids, (0, extra), value=pad_id),
                torch.nn.functional.pad(mask, (0, extra), value=0))

    a_ids, a_mask = pad(a_ids, a_mask)
    b_ids, b_mask = pad(b_ids, b_mask)
    return a_ids, a_mask, b_ids, b_mask


class ARPipelineExecutorBase:
    family: str
    task: str
    default_image_token_num: int | None = 576
    default_image_size: int | None = 384
    default_max_text_length: int | None = 256

    def parse_spec(self, request: GenerationRequest) -> ARGenerationSpec:
        return parse_ar_generation_spec(
            request, default_image_token_num=self.default_image_token_num,
            default_image_size=self.default_image_size,
            default_max_text_length=self.default_max_text_length)

    def expand_prompts(self, request): return expand_prompt_major_prompts(request)
    def validate_chunk(self, request, chunk): validate_chunk(request, chunk)
    def require_rows(self, name, value, count): require_rows(name, value, count)
    def chunk_seed_offset(self, request, chunk): return chunk_seed_offset(request, chunk)
    def max_peak_memory_mb(self, chunks): return max_peak_memory_mb(chunks)
    def peak_memory_mb(self): return peak_memory_mb()

    def ordered_chunks(self, request, sample_specs, chunks, *, row_fields=()):
        return ordered_chunks(request, sample_specs, chunks, row_fields=row_fields)

    def align_pair(self, a_ids, a_mask, b_ids, b_mask, pad_id: int = 0):
        return align_pair(a_ids, a_mask, b_ids, b_mask, pad_id=pad_id)

    def forward_batch(self, requests, sample_specs_by_request) -> dict[str, OutputBatch]:
        return forward_batch_by_merging_prompts(self, requests, sample_specs_by_request)


__all__ = [
    "ARChunkResult", "ARPipelineExecutorBase", "align_pair", "chunk_seed_offset",
    "expand_prompt_major_prompts", "max_peak_memory_mb", "ordered_chunks",
    "parse_ar_generation_spec", "peak_memory_mb", "require_rows", "validate_chunk",
]
