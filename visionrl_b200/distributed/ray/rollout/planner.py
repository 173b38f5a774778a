"""Which worker runs which chunk of a request.

The chunk list is the prompt-major micro-batch plan of the request (chunks of at most
``sampling.sample_batch_size`` samples of one prompt); workers are dealt chunks in turn, the same
round-robin deal the SPMD runtime uses over its data-parallel ranks
(:meth:`visionrl_b200.engine.microbatching.ExecutionPlan.for_rank`), so a pool of ``n`` workers
and a job of ``n`` ranks cut a request identically.  The result is listed in plan order, which is
the order results must be gathered in.  Behavioural reference:
``vrl/distributed/ray/rollout/planner.py:15-54``.
"""

from __future__ import annotations

from dataclasses import dataclass

from visionrl_b200.distributed.ray.rollout.types import RayWorkerHandle
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.microbatching import (
    ExecutionPlan, MicroBatchPlan, plan_prompt_group_microbatches,
)


@dataclass(frozen=True, slots=True)
class DeviceAssignment:
    worker_id: str
    node_id: str
    gpu_ids: tuple[int, ...]
    chunk: MicroBatchPlan


def request_chunks(request: GenerationRequest) -> ExecutionPlan:
    """The micro-batch plan every consumer of ``request`` derives (no state, no communication)."""
    cap = int(request.sampling.get("sample_batch_size", request.samples_per_prompt))
    return plan_prompt_group_microbatches(request.prompts, request.samples_per_prompt, max(1, cap))


class DistributedExecutionPlanner:
    def plan_by_worker(self, request: GenerationRequest,
                       workers: list[RayWorkerHandle]) -> dict[str, tuple[MicroBatchPlan, ...]]:
        if not workers:
            raise ValueError("DistributedExecutionPlanner requires at least one worker")
        plan = request_chunks(request)
        return {w.worker_id: plan.for_rank(i, len(workers)) for i, w in enumerate(workers)}

    def plan(self, request: GenerationRequest, workers: list[RayWorkerHandle]) -> list[DeviceAssignment]:
        dealt = self.plan_by_worker(request, workers)
        by_chunk = {id(chunk): w for w in workers for chunk in dealt[w.worker_id]}
        ordered = sorted((c for cs in dealt.values() for c in cs),
                         key=lambda c: (c.prompt_index, c.sample_start))
        return [DeviceAssignment(w.worker_id, w.node_id, w.gpu_ids, c)
                for c in ordered for w in (by_chunk[id(c)],)]


__all__ = ["DeviceAssignment", "DistributedExecutionPlanner", "request_chunks"]
