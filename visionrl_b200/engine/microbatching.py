"""Micro-batch plans of a rollout request and their execution under memory pressure.

A request of ``P`` prompts × ``G`` samples is cut into *chunks*: runs of at most
``max_samples_per_microbatch`` samples of ONE prompt, listed prompt-major, so a GRPO group is
always a contiguous run of chunks.  The same list serves three consumers:

* a single executor walks it front to back;
* the SPMD runtime deals it round-robin over the data-parallel ranks (:meth:`ExecutionPlan.for_rank`)
  — every rank computes the same plan from the same request, so no assignment is ever sent;
* the worker-pool facade deals it round-robin over its workers.

:class:`BisectingRunner` executes chunks and, when one fails with a CUDA out-of-memory error,
frees the allocator cache and retries it as two halves (left half first) down to
``min_sample_count`` samples.  It records which chunk each result came from, because after a
bisection the results no longer line up one-to-one with the plan and the caller has to know which
samples each result holds.  Behavioural reference: ``vrl/engine/microbatching.py:12-154``.
"""

from __future__ import annotations

from collections.abc import Callable, Iterable, Sequence
from dataclasses import dataclass, field
from typing import Generic, TypeVar

T = TypeVar("T")


@dataclass(frozen=True, slots=True)
class MicroBatchPlan:
    """Samples ``[sample_start, sample_start + sample_count)`` of prompt ``prompt_index``."""

    prompt_index: int
    prompt: str
    sample_start: int
    sample_count: int

    def __post_init__(self) -> None:
        for name, floor in (("prompt_index", 0), ("sample_start", 0), ("sample_count", 1)):
            if getattr(self, name) < floor:
                raise ValueError(f"{name} must be >= {floor}")

    @property
    def sample_end(self) -> int:
        return self.sample_start + self.sample_count

    def split(self) -> tuple["MicroBatchPlan", "MicroBatchPlan"]:
        """Two halves covering the same samples; the left one is the smaller when odd."""
        if self.sample_count <= 1:
            raise ValueError("Cannot split a single-sample micro-batch")
        left = self.sample_count // 2
        return (MicroBatchPlan(self.prompt_index, self.prompt, self.sample_start, left),
                MicroBatchPlan(self.prompt_index, self.prompt, self.sample_start + left,
                               self.sample_count - left))


@dataclass(frozen=True, slots=True)
class ExecutionPlan:
    prompts: tuple[str, ...]
    samples_per_prompt: int
    max_samples_per_microbatch: int
    micro_batches: tuple[MicroBatchPlan, ...]

    @property
    def total_samples(self) -> int:
        return len(self.prompts) * self.samples_per_prompt

    def for_rank(self, rank: int, world: int) -> tuple[MicroBatchPlan, ...]:
        """The chunks member ``rank`` of ``world`` equal consumers runs (round-robin deal)."""
        if world < 1 or not 0 <= rank < world:
            raise ValueError(f"rank {rank} is outside a group of {world}")
        return self.micro_batches[rank::world]


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
    chunks: list[MicroBatchPlan] = []
    for index, prompt in enumerate(prompts):
        start = 0
        while start < samples_per_prompt:
            count = min(max_samples_per_microbatch, samples_per_prompt - start)
            chunks.append(MicroBatchPlan(index, prompt, start, count))
            start += count
    return ExecutionPlan(tuple(prompts), int(samples_per_prompt), int(max_samples_per_microbatch),
                         tuple(chunks))


def is_cuda_oom(exc: BaseException) -> bool:
    """True for the allocator's ``RuntimeError`` (``torch.cuda.OutOfMemoryError`` is one)."""
    text = str(exc).lower()
    return "cuda" in text and "out of memory" in text


def _drop_allocator_cache() -> None:
    try:
        import torch

        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    except Exception:  # noqa: BLE001 - best effort; the retry happens either way
        pass


@dataclass
class BisectingRunner(Generic[T]):
    """Runs chunks through ``run_one``; an out-of-memory chunk is retried as two halves.

    ``results[i]`` was produced by ``executed[i]``; ``bisections`` counts the splits.
    """

    run_one: Callable[[MicroBatchPlan], T]
    min_sample_count: int = 1
    results: list[T] = field(default_factory=list)
    executed: list[MicroBatchPlan] = field(default_factory=list)
    bisections: int = 0

    def __post_init__(self) -> None:
        if self.min_sample_count < 1:
            raise ValueError("min_sample_count must be >= 1")

    def run(self, chunks: Iterable[MicroBatchPlan]) -> list[T]:
        # depth-first over the bisection tree keeps the results in sample order
        stack = list(chunks)[::-1]
        while stack:
            chunk = stack.pop()
            try:
                value = self.run_one(chunk)
            except RuntimeError as exc:
                if not is_cuda_oom(exc) or chunk.sample_count <= self.min_sample_count:
                    raise
                _drop_allocator_cache()
                left, right = chunk.split()
                stack.extend((right, left))
                self.bisections += 1
                continue
            self.results.append(value)
            self.executed.append(chunk)
        return self.results


def run_microbatches_with_oom_retry(micro_batches: Sequence[MicroBatchPlan],
                                    run_one: Callable[[MicroBatchPlan], T], *,
                                    min_sample_count: int = 1) -> list[T]:
    """Results of every chunk in sample order, bisecting chunks that run out of device memory."""
    return BisectingRunner(run_one, min_sample_count).run(micro_batches)


__all__ = [
    "BisectingRunner", "ExecutionPlan", "MicroBatchPlan", "RolloutShardPlan", "is_cuda_oom",
    "plan_prompt_group_microbatches", "run_microbatches_with_oom_retry",
]
