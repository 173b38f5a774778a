"""In-process rollout backend (reference: ``vrl/engine/core/runtime.py:12-56``)."""

from __future__ import annotations

import asyncio
from typing import Protocol

from visionrl_b200.engine.core.types import GenerationRequest, OutputBatch
from visionrl_b200.engine.core.worker import GenerationWorker


class RolloutBackend(Protocol):
    async def generate(self, request: GenerationRequest) -> OutputBatch: ...


class GenerationRuntime(RolloutBackend):
    def __init__(self, worker: GenerationWorker, *, execute_in_thread: bool = False) -> None:
        self.worker = worker
        self.execute_in_thread = execute_in_thread

    async def generate(self, request: GenerationRequest) -> OutputBatch:
        outputs = await self.generate_many([request])
        found = outputs.get(request.request_id)
        if found is not None:
            return found
        return OutputBatch(
            request_id=request.request_id, family="unknown", task="unknown", prompts=[],
            sample_specs=[], output=None,
            error="Generation worker did not return an output for this request",
        )

    async def generate_many(self, requests: list[GenerationRequest]) -> dict[str, OutputBatch]:
        if self.execute_in_thread:
            loop = asyncio.get_running_loop()
            return await loop.run_in_executor(None, self.worker.execute, requests)
        return self.worker.execute(requests)

    async def shutdown(self) -> None:
        return None
