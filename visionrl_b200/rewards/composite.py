"""Weighted sum of reward functions.

The member rewards are independent of one another, so a batch is scored by all of them
concurrently (``asyncio.gather``): a remote scorer's round trip overlaps a tower running on the
device.  The result is the same weighted sum the reference computes member by member
(``vrl/rewards/composite.py:9-28``).
"""

from __future__ import annotations

import asyncio
from typing import Sequence

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction


class CompositeReward(RewardFunction):
    def __init__(self, rewards: Sequence[tuple[float, RewardFunction]]) -> None:
        self.rewards = list(rewards)

    async def score(self, rollout: Rollout) -> float:
        return (await self.score_batch([rollout]))[0]

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        if not self.rewards:
            return [0.0] * len(rollouts)
        columns = await asyncio.gather(*(fn.score_batch(rollouts) for _, fn in self.rewards))
        weights = [float(w) for w, _ in self.rewards]
        for (_, fn), column in zip(self.rewards, columns):
            if len(column) != len(rollouts):
                raise ValueError(f"{type(fn).__name__}.score_batch returned {len(column)} scores "
                                 f"for {len(rollouts)} rollouts")
        return [sum(w * float(col[i]) for w, col in zip(weights, columns)) for i in range(len(rollouts))]
