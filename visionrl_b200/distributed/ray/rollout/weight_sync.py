"""Pushes a trainable state and its policy version to every rollout worker
(reference: ``vrl/distributed/ray/rollout/weight_sync.py:12-48``)."""

from __future__ import annotations

import asyncio
from typing import Any, Protocol

from visionrl_b200.distributed.ray.rollout.types import RayWorkerHandle


class RolloutWeightSync(Protocol):
    """What a runtime needs from its weight channel: push a trainable state with its version."""

    async def push_to_rollout_workers(self, state_ref: Any, policy_version: int) -> None: ...


class RayRolloutWeightSync:
    def __init__(self, workers: list[RayWorkerHandle]) -> None:
        self.workers = list(workers)

    async def push_to_rollout_workers(self, state_ref: Any, policy_version: int) -> None:
        refs = []
        for w in self.workers:
            fn = w.actor.update_weights
            remote = getattr(fn, "remote", None)
            if callable(remote):
                refs.append(remote(state_ref, policy_version))
            else:
                fn(state_ref, policy_version)
        if refs:
            from visionrl_b200.distributed.ray.dependencies import require_ray

            await asyncio.to_thread(require_ray().get, refs)


__all__ = ["RayRolloutWeightSync", "RolloutWeightSync"]
