"""Named, weighted reward mix with per-component history
(reference: ``vrl/rewards/multi.py:15-116``).

``last_components[name]`` accumulates raw component scores of every call since the last
``reset_components()`` so a training loop can log component means per step.
"""

from __future__ import annotations

import inspect
from typing import Any

import torch

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction

_REWARD_REGISTRY: dict[str, type[RewardFunction]] = {}


def register_reward(name: str, cls: type[RewardFunction]) -> None:
    _REWARD_REGISTRY[name] = cls


def get_reward(name: str) -> type[RewardFunction]:
    if name not in _REWARD_REGISTRY:
        raise KeyError(f"Unknown reward function: {name!r}. Available: {list(_REWARD_REGISTRY)}")
    return _REWARD_REGISTRY[name]


def _register_builtins() -> None:
    from visionrl_b200.rewards.aesthetic import AestheticReward
    from visionrl_b200.rewards.clip import CLIPScoreReward
    from visionrl_b200.rewards.ocr import OCRReward
    from visionrl_b200.rewards.pickscore import PickScoreReward
    from visionrl_b200.rewards.synthetic import LatentTargetReward, ViTScalarReward

    for name, cls in (("aesthetic", AestheticReward), ("clipscore", CLIPScoreReward),
                      ("ocr", OCRReward), ("pickscore", PickScoreReward),
                      ("vit_scalar", ViTScalarReward), ("latent_target", LatentTargetReward)):
        _REWARD_REGISTRY.setdefault(name, cls)


class MultiReward(RewardFunction):
    def __init__(self, rewards: list[tuple[str, float, RewardFunction]]) -> None:
        self.rewards = rewards
        self.last_components: dict[str, list[float]] = {}
        self.last_component_tensors: dict[str, list[torch.Tensor]] = {}

    def reset_components(self) -> None:
        self.last_components = {}
        self.last_component_tensors = {}

    @classmethod
    def from_dict(cls, score_dict: dict[str, float], device: str = "cuda",
                  reward_kwargs: dict[str, dict[str, Any]] | None = None) -> "MultiReward":
        _register_builtins()
        reward_kwargs = reward_kwargs or {}
        return cls([(name, weight, get_reward(name)(device=device, **(reward_kwargs.get(name) or {})))
                    for name, weight in score_dict.items()])

    def _record(self, components: dict[str, list[float]]) -> None:
        for name, values in components.items():
            self.last_components.setdefault(name, []).extend(float(v) for v in values)

    async def score(self, rollout: Rollout) -> float:
        total, components = 0.0, {}
        for name, weight, fn in self.rewards:
            s = await fn.score(rollout)
            components[name] = [s]
            total += weight * s
        self._record(components)
        return total

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        totals = [0.0] * len(rollouts)
        components: dict[str, list[float]] = {}
        for name, weight, fn in self.rewards:
            scores = await fn.score_batch(rollouts)
            components[name] = list(scores)
            for i, s in enumerate(scores):
                totals[i] += weight * s
        self._record(components)
        return totals

    async def score_tensor_batch(self, outputs, prompts, metadata):
        """Device-side scoring when every component supports it; ``None`` otherwise (the
        caller then falls back to ``score_batch``).  Component histories are kept as device
        tensors in ``last_component_tensors`` and folded into ``last_components`` lazily by
        :meth:`component_means`."""
        if not all(hasattr(fn, "score_tensor_batch") for _, _, fn in self.rewards):
            return None
        total = None
        for name, weight, fn in self.rewards:
            s = fn.score_tensor_batch(outputs, prompts, metadata)
            if inspect.isawaitable(s):
                s = await s
            s = s.float()
            self.last_component_tensors.setdefault(name, []).append(s.detach())
            total = weight * s if total is None else total + weight * s
        return total

    def component_means(self) -> dict[str, float]:
        out = {}
        names = set(self.last_components) | set(self.last_component_tensors)
        for name in names:
            vals = list(self.last_components.get(name, []))
            tensors = self.last_component_tensors.get(name, [])
            if tensors:
                vals.extend(torch.cat([t.reshape(-1) for t in tensors]).tolist())
            out[name] = sum(vals) / len(vals) if vals else 0.0
        return out
