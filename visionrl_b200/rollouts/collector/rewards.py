"""Reward scoring of generated outputs.

Reward functions that implement ``score_tensor_batch(outputs, prompts, metadata)``
score the whole device-resident batch in one call and return a device tensor;
all others receive one ``Rollout`` per sample through ``score_batch`` / ``score``
(reference: ``vrl/rollouts/collector/rewards.py:14-61``).  Without a reward
function the scores are zeros.
"""

from __future__ import annotations

import inspect
from collections.abc import Mapping, Sequence
from typing import Any

import torch

from visionrl_b200.algorithms.types import Rollout, Trajectory


def _rows(outputs: Any) -> int:
    shape = getattr(outputs, "shape", None)
    return int(shape[0]) if shape is not None else len(outputs)


class RewardScorer:
    def __init__(self, reward_fn: Any | None) -> None:
        self.reward_fn = reward_fn

    async def score(self, outputs: Any, prompts: Sequence[str], metadata: Mapping[str, Any],
                    device: Any) -> torch.Tensor:
        n = _rows(outputs)
        if self.reward_fn is None:
            return torch.zeros(n, device=device)
        fused = getattr(self.reward_fn, "score_tensor_batch", None)
        if fused is not None:
            raw = fused(outputs, list(prompts), dict(metadata))
            if inspect.isawaitable(raw):
                raw = await raw
            if raw is not None:
                return torch.as_tensor(raw, dtype=torch.float32).to(device)
        rollouts = [
            Rollout(request=None,
                    trajectory=Trajectory(prompt=prompts[i], seed=0, steps=[], output=outputs[i]),
                    metadata=dict(metadata))
            for i in range(n)
        ]
        batch_fn = getattr(self.reward_fn, "score_batch", None)
        if batch_fn is not None:
            raw = batch_fn(rollouts)
            if inspect.isawaitable(raw):
                raw = await raw
        else:
            raw = []
            for r in rollouts:
                value = self.reward_fn.score(r)
                raw.append(await value if inspect.isawaitable(value) else value)
        return torch.tensor([float(x) for x in raw], device=device, dtype=torch.float32)


__all__ = ["RewardScorer"]
