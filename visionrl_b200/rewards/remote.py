"""Reward served over HTTP: POST ``{prompt, seed, reward, metadata}`` and read ``score`` (or
``scores`` for a batch) from the JSON reply (reference: ``vrl/rewards/remote.py:13-49``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction


class RemoteReward(RewardFunction):
    def __init__(self, url: str, timeout: float | None = None, reward_name: str = "default",
                 timeout_s: float = 60.0, session: Any | None = None) -> None:
        # ``timeout`` (seconds) is the reference's name and position for the request time limit
        self.url, self.reward_name = url, reward_name
        self.timeout_s = float(timeout) if timeout is not None else float(timeout_s)
        self._session = session

    def _payload(self, rollout: Rollout) -> dict[str, Any]:
        return {"prompt": rollout.trajectory.prompt, "seed": rollout.trajectory.seed,
                "reward": self.reward_name, "metadata": dict(rollout.metadata)}

    async def _post(self, payload: dict[str, Any]) -> dict[str, Any]:
        import aiohttp

        if self._session is not None:
            async with self._session.post(self.url, json=payload) as resp:
                resp.raise_for_status()
                return await resp.json()
        timeout = aiohttp.ClientTimeout(total=self.timeout_s)
        async with aiohttp.ClientSession(timeout=timeout) as session:
            async with session.post(self.url, json=payload) as resp:
                resp.raise_for_status()
                return await resp.json()

    async def score(self, rollout: Rollout) -> float:
        return float((await self._post(self._payload(rollout)))["score"])

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        reply = await self._post({"reward": self.reward_name,
                                  "items": [self._payload(r) for r in rollouts]})
        if "scores" in reply:
            return [float(s) for s in reply["scores"]]
        return [await self.score(r) for r in rollouts]
