"""Weighted sum of reward functions (reference: ``vrl/rewards/composite.py:9-28``)."""

from __future__ import annotations

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction


class CompositeReward(RewardFunction):
    def __init__(self, rewards: list[tuple[float, RewardFunction]]) -> None:
        self.rewards = rewards

    async def score(self, rollout: Rollout) -> float:
        total = 0.0
        for weight, fn in self.rewards:
            total += weight * await fn.score(rollout)
        return total

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        totals = [0.0] * len(rollouts)
        for weight, fn in self.rewards:
            for i, s in enumerate(await fn.score_batch(rollouts)):
                totals[i] += weight * s
        return totals
