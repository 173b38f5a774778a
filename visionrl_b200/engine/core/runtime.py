"""The rollout-backend contract and its in-process implementation.

Every rollout backend of this package — this one, the SPMD runtime that deals chunks over the
ranks of a job, the worker-pool facade — answers ``await generate(request)`` with an
``OutputBatch`` and, when it can be told about new weights, ``await update_weights(state,
version)``.  A backend that tracks a policy version refuses a request stamped with another one:
training on samples of stale weights is the failure this guards against.

``GenerationRuntime`` runs requests through one ``GenerationWorker`` in the calling process
(optionally on a helper thread so an event loop stays responsive).  It shares the executor's
model with the trainer by construction, so a weight update only has to move the version forward.
Behavioural reference: ``vrl/engine/core/runtime.py:12-56``.
"""

from __future__ import annotations

import asyncio
import dataclasses
from typing import Any, Protocol

from visionrl_b200.engine.core.types import GenerationRequest, OutputBatch
from visionrl_b200.engine.core.worker import GenerationWorker


class RolloutBackend(Protocol):
    async def generate(self, request: GenerationRequest) -> OutputBatch: ...


def stamp_policy_version(request: GenerationRequest, current: int | None) -> GenerationRequest:
    """``request`` carrying the backend's version; ``RuntimeError`` when it asks for another."""
    if current is None or request.policy_version == current:
        return request
    if request.policy_version is None:
        return dataclasses.replace(request, policy_version=current)
    raise RuntimeError(f"policy_version mismatch: expected={request.policy_version}, "
                       f"actual={current}")


def unanswered(request: GenerationRequest) -> OutputBatch:
    return OutputBatch(request_id=request.request_id, family="unknown", task="unknown", prompts=[],
                       sample_specs=[], output=None,
                       error="Generation worker did not return an output for this request")


class GenerationRuntime(RolloutBackend):
    def __init__(self, worker: GenerationWorker, *, execute_in_thread: bool = False,
                 policy_version: int | None = None) -> None:
        self.worker = worker
        self.execute_in_thread = execute_in_thread
        self.current_policy_version = policy_version
        self.shares_trainer_weights = True

    async def generate_many(self, requests: list[GenerationRequest]) -> dict[str, OutputBatch]:
        """Outputs by request id; same-config requests may be fused by the worker."""
        stamped = [stamp_policy_version(r, self.current_policy_version) for r in requests]
        if self.execute_in_thread:
            return await asyncio.to_thread(self.worker.execute, stamped)
        return self.worker.execute(stamped)

    async def generate(self, request: GenerationRequest) -> OutputBatch:
        answers = await self.generate_many([request])
        return answers.get(request.request_id) or unanswered(request)

    async def update_weights(self, state_ref: Any, policy_version: int) -> None:
        """The worker's executor reads the caller's live model; only the version moves."""
        del state_ref
        self.current_policy_version = int(policy_version)

    async def shutdown(self) -> None:
        return None


__all__ = ["GenerationRuntime", "RolloutBackend", "stamp_policy_version", "unanswered"]
