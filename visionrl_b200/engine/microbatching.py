"""Prompt-major micro-batch planning and out-of-memory bisection
(reference: ``vrl/engine/microbatching.py:12-154``).

A plan never mixes prompts inside a micro-batch, so GRPO groups stay contiguous.
When a micro-batch raises a CUDA out-of-memory ``RuntimeError`` it is halved
(left half first) until ``min_sample_count`` is reached.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Callable, Sequence
from dataclasses import dataclass
from typing import TypeVar

T = TypeVar("T")


@dataclass(frozen=True, slots=True)
class MicroBatchPlan:
    prompt_index: int
    prompt: str
    sample_start: int
    sample_count: int

    def __post_init__(self) -> None:
        if self.prompt_index < 0:
            raise ValueError("prompt_index must be >= 0")
        if self.sample_start < 0:
            raise ValueError("sample_start must be >= 0")
        if self.sample_count < 1:
            raise ValueError("sample_count must be >= 1")

    @property
    def sample_end(self) -> int:
        return self.sample_start + self.sample_count

    def split(self) -> tuple["MicroBatchPlan", "MicroBatchPlan"]:
        if self.sample_count <= 1:
            raise ValueError("Cannot split a single-sample micro-batch")
        head = self.sample_count // 2
        return (
            MicroBatchPlan(self.prompt_index, self.prompt, self.sample_start, head),
            MicroBatchPlan(self.prompt_index, self.prompt, self.sample_start + head,
                           self.sample_count - head),
        )


@dataclass(frozen=True, slots=True)
class ExecutionPlan:
    prompts: tuple[str, ...]
    samples_per_prompt: int
    max_samples_per_microbatch: int
    micro_batches: tuple[MicroBatchPlan, ...]

    @property
    def total_samples(self) -> int:
        return len(self.prompts) * self.samples_per_prompt


@dataclass(frozen=True, slots=True)
class RolloutShardPlan:
    request_id: str
    chunks: tuple[MicroBatchPlan, ...]


def plan_prompt_group_microbatches(prompts: Sequence[str], samples_per_prompt: int,
                                   max_samples_per_microbatch: int) -> ExecutionPlan:
    if not prompts:
        raise ValueError("prompts must be non-empty")
    if samples_per_prompt < 1:
        raise ValueError("samples_per_prompt must be >= 1")
    if max_samples_per_microbatch < 1:
        raise ValueError("max_samples_per_microbatch must be >= 1")
    plans = [
        MicroBatchPlan(i, prompt, start, min(max_samples_per_microbatch, samples_per_prompt - start))
        for i, prompt in enumerate(prompts)
        for start in range(0, samples_per_prompt, max_samples_per_microbatch)
    ]
    return ExecutionPlan(tuple(prompts), samples_per_prompt, max_samples_per_microbatch,
                         tuple(plans))


def is_cuda_oom(exc: BaseException) -> bool:
    text = str(exc).lower()
    return "cuda" in text and "out of memory" in text


def run_microbatches_with_oom_retry(micro_batches: Sequence[MicroBatchPlan],
                                    run_one: Callable[[MicroBatchPlan], T], *,
                                    min_sample_count: int = 1) -> list[T]:
    if min_sample_count < 1:
        raise ValueError("min_sample_count must be >= 1")
    queue = deque(micro_batches)
    done: list[T] = []
    while queue:
        plan = queue.popleft()
        try:
            done.append(run_one(plan))
        except RuntimeError as exc:
            if not is_cuda_oom(exc) or plan.sample_count <= min_sample_count:
                raise
            try:
                import torch

                if torch.cuda.is_available():
                    torch.cuda.empty_cache()
            except Exception:  # noqa: BLE001
                pass
            queue.extendleft(reversed(plan.split()))
    return done


__all__ = [
    "ExecutionPlan", "MicroBatchPlan", "RolloutShardPlan", "is_cuda_oom",
    "plan_prompt_group_microbatches", "run_microbatches_with_oom_retry",
]
