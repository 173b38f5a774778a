"""Chunk → worker assignment: prompt-major micro-batches of ``sample_batch_size``
handed out round-robin (reference: ``vrl/distributed/ray/rollout/planner.py:15-54``)."""

from __future__ import annotations

from dataclasses import dataclass

from visionrl_b200.distributed.ray.rollout.types import RayWorkerHandle
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.microbatching import MicroBatchPlan, plan_prompt_group_microbatches


@dataclass(frozen=True, slots=True)
class DeviceAssignment:
    worker_id: str
    node_id: str
    gpu_ids: tuple[int, ...]
    chunk: MicroBatchPlan


class DistributedExecutionPlanner:
    def plan(self, request: GenerationRequest, workers: list[RayWorkerHandle]) -> list[DeviceAssignment]:
        if not workers:
            raise ValueError("DistributedExecutionPlanner requires at least one worker")
        cap = int(request.sampling.get("sample_batch_size", request.samples_per_prompt))
        plan = plan_prompt_group_microbatches(request.prompts, request.samples_per_prompt,
                                              max(1, cap))
        return [
            DeviceAssignment(w.worker_id, w.node_id, w.gpu_ids, chunk)
            for i, chunk in enumerate(plan.micro_batches)
            for w in (workers[i % len(workers)],)
        ]


__all__ = ["DeviceAssignment", "DistributedExecutionPlanner"]
