"""Rewards for synthetic-data runs.

* ``ViTScalarReward`` — a ViT tower (``vit_l14`` / ``vit_b16`` preset) with a scalar head,
  applied to the decoded image or to ``num_frames`` evenly spaced video frames.
* ``LatentTargetReward`` — negative mean squared distance of the final output to a
  seed-fixed ``N(0, 1)`` target of the same shape.
"""

from __future__ import annotations

import torch

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction
from visionrl_b200.rewards.vision_tower import build_image_tower, frames_for_scoring


class ViTScalarReward(RewardFunction):
    def __init__(self, device: str = "cuda", preset: str = "vit_l14", seed: int = 0,
                 num_frames: int = 4, batch_size: int = 64) -> None:
        self._device, self.preset, self.seed = device, preset, seed
        self.num_frames, self.batch_size = num_frames, batch_size
        self._tower = None

    def _ensure_loaded(self) -> None:
        if self._tower is None:
            self._tower = build_image_tower(f"random:{self.preset}:{self.seed}", self._device)

    @torch.no_grad()
    def score_tensor_batch(self, outputs: torch.Tensor, prompts=None, metadata=None) -> torch.Tensor:
        self._ensure_loaded()
        k = self.num_frames
        fractions = tuple((i + 0.5) / k for i in range(k))
        frames = frames_for_scoring(outputs.to(self._device), fractions)
        b, kk = frames.shape[:2]
        flat = frames.reshape(b * kk, *frames.shape[2:])
        scores = torch.cat([self._tower(flat[i:i + self.batch_size])
                            for i in range(0, flat.shape[0], self.batch_size)])
        return scores.view(b, kk).mean(dim=1)

    async def score(self, rollout: Rollout) -> float:
        return float(self.score_tensor_batch(rollout.trajectory.output.unsqueeze(0))[0])

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        return self.score_tensor_batch(torch.stack([r.trajectory.output for r in rollouts])).tolist()


class LatentTargetReward(RewardFunction):
    def __init__(self, device: str = "cpu", seed: int = 0) -> None:
        self._device, self.seed = device, seed
        self._targets: dict[tuple, torch.Tensor] = {}

    def _target(self, shape: tuple, device) -> torch.Tensor:
        if shape not in self._targets:
            g = torch.Generator().manual_seed(self.seed + 104729)
            self._targets[shape] = torch.randn(shape, generator=g)
        return self._targets[shape].to(device)

    @torch.no_grad()
    def score_tensor_batch(self, outputs: torch.Tensor, prompts=None, metadata=None) -> torch.Tensor:
        x = outputs.float()
        target = self._target(tuple(x.shape[1:]), x.device)
        return -((x - target) ** 2).mean(dim=tuple(range(1, x.ndim)))

    async def score(self, rollout: Rollout) -> float:
        return float(self.score_tensor_batch(rollout.trajectory.output.unsqueeze(0))[0])
