"""Reward function interface (reference: ``vrl/rewards/base.py:10-19``).

``score`` rates one rollout; ``score_batch`` defaults to a sequential loop.  Model-backed
rewards additionally implement ``score_tensor_batch(outputs, prompts, metadata)`` which
scores a device-resident batch in one forward and returns a device tensor.
"""

from __future__ import annotations

from abc import ABC, abstractmethod

from visionrl_b200.algorithms.types import Rollout


class RewardFunction(ABC):
    @abstractmethod
    async def score(self, rollout: Rollout) -> float: ...

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        return [await self.score(r) for r in rollouts]
