"""Collector protocol (reference: ``vrl/rollouts/collector/base.py``)."""

from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

from visionrl_b200.rollouts.batch import RolloutBatch


@runtime_checkable
class Collector(Protocol):
    async def collect(self, prompts: list[str], **kwargs: Any) -> RolloutBatch: ...
