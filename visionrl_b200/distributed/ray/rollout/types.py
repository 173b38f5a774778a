"""Worker handle and chunk result envelope (reference: ``vrl/distributed/ray/rollout/types.py:12-32``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from visionrl_b200.engine.core.protocols import PipelineChunkResult
from visionrl_b200.engine.microbatching import MicroBatchPlan


@dataclass(slots=True)
class RayWorkerHandle:
    worker_id: str
    node_id: str
    gpu_ids: tuple[int, ...] = ()
    actor: Any | None = None


@dataclass(slots=True)
class RayChunkResult:
    request_id: str
    worker_id: str
    chunk: MicroBatchPlan
    output: PipelineChunkResult | None
    metrics: dict[str, Any] = field(default_factory=dict)
    policy_version: int | None = None
    error: str | None = None


__all__ = ["RayChunkResult", "RayWorkerHandle"]
