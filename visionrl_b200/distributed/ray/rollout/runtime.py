"""Runtime facade over executor + weight sync (reference: ``vrl/distributed/ray/rollout/runtime.py:17-72``)."""

from __future__ import annotations

import dataclasses
from typing import Any

from visionrl_b200.distributed.ray.rollout.executor import DistributedRolloutExecutor
from visionrl_b200.distributed.ray.rollout.types import RayWorkerHandle
from visionrl_b200.distributed.ray.rollout.weight_sync import RayRolloutWeightSync
from visionrl_b200.engine.core.types import GenerationRequest, OutputBatch


class RayDistributedRuntime:
    def __init__(self, executor: DistributedRolloutExecutor, workers: list[RayWorkerHandle] | None = None,
                 weight_sync: RayRolloutWeightSync | None = None, placement_group: Any | None = None,
                 policy_version: int | None = None, *,
                 owned_workers: list[RayWorkerHandle] | None = None) -> None:
        # ``owned_workers`` is the reference's keyword for the workers this runtime shuts down
        workers = owned_workers if workers is None else workers
        self.executor, self.workers, self.weight_sync = executor, list(workers or []), weight_sync
        self.placement_group = placement_group
        self.current_policy_version = policy_version

    async def generate(self, request: GenerationRequest) -> OutputBatch:
        if request.policy_version is None and self.current_policy_version is not None:
            request = dataclasses.replace(request, policy_version=self.current_policy_version)
        return await self.executor.execute(request)

    async def update_weights(self, state_ref: Any, policy_version: int) -> None:
        if self.weight_sync is None:
            raise RuntimeError("runtime was launched with sync_trainable_state='disabled'")
        await self.weight_sync.push_to_rollout_workers(state_ref, int(policy_version))
        self.current_policy_version = int(policy_version)

    async def shutdown(self) -> None:
        for w in self.workers:
            release = getattr(w.actor, "release_policy", None)
            if callable(release) and not callable(getattr(release, "remote", None)):
                release()
            w.actor = None
        if self.placement_group is not None:
            self.placement_group.remove()
            self.placement_group = None


__all__ = ["RayDistributedRuntime"]
