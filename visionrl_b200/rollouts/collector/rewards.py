"""Turning generated outputs into one reward per sample.

The outputs of a rollout (decoded images or frames) are already a device tensor when they reach
this point, so the preferred route is a reward that scores the whole batch where it lies:
``score_tensor_batch(outputs, prompts, metadata) -> [B]``.  Rewards without that method are fed
the reference's per-sample ``Rollout`` objects, through ``score_batch`` when they have it and one
``score`` call per sample otherwise; either may be a coroutine function.  Whatever the route, the
answer is an fp32 ``[B]`` tensor on the requested device — zeros when no reward is configured.
Behavioural reference: ``vrl/rollouts/collector/rewards.py:14-61``.
"""

from __future__ import annotations

import inspect
from collections.abc import Mapping, Sequence
from typing import Any

import torch

from visionrl_b200.algorithms.types import Rollout, Trajectory


async def _settled(value: Any) -> Any:
    return await value if inspect.isawaitable(value) else value


def _batch_size(outputs: Any) -> int:
    shape = getattr(outputs, "shape", None)
    return int(shape[0]) if shape is not None else len(outputs)


def as_rollouts(outputs: Any, prompts: Sequence[str], metadata: Mapping[str, Any]) -> list[Rollout]:
    """One reference-style ``Rollout`` per sample (what per-sample reward functions consume)."""
    return [Rollout(request=None, metadata=dict(metadata),
                    trajectory=Trajectory(prompt=prompts[i], seed=0, steps=[], output=outputs[i]))
            for i in range(_batch_size(outputs))]


class RewardScorer:
    def __init__(self, reward_fn: Any | None) -> None:
        self.reward_fn = reward_fn

    async def _whole_batch(self, outputs, prompts, metadata) -> Any | None:
        fn = getattr(self.reward_fn, "score_tensor_batch", None)
        if fn is None:
            return None
        return await _settled(fn(outputs, list(prompts), dict(metadata)))

    async def _per_sample(self, outputs, prompts, metadata) -> list[float]:
        rollouts = as_rollouts(outputs, prompts, metadata)
        batched = getattr(self.reward_fn, "score_batch", None)
        if batched is not None:
            return [float(v) for v in await _settled(batched(rollouts))]
        return [float(await _settled(self.reward_fn.score(r))) for r in rollouts]

    async def score(self, outputs: Any, prompts: Sequence[str], metadata: Mapping[str, Any],
                    device: Any) -> torch.Tensor:
        if self.reward_fn is None:
            return torch.zeros(_batch_size(outputs), device=device)
        scores = await self._whole_batch(outputs, prompts, metadata)
        if scores is None:
            scores = await self._per_sample(outputs, prompts, metadata)
        return torch.as_tensor(scores, dtype=torch.float32).to(device)


__all__ = ["RewardScorer", "as_rollouts"]
