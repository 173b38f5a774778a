"""Aesthetic predictor: L2-normalised ViT-L/14 image features → MLP
``768→1024→128→64→16→1``; videos average the frames at 25/50/75 %
(reference: ``vrl/rewards/aesthetic.py:15-121``)."""

from __future__ import annotations

import torch
from torch import nn

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction
from visionrl_b200.rewards.vision_tower import build_image_tower, frames_for_scoring


class AestheticMLP(nn.Module):
    def __init__(self, in_dim: int = 768):
        super().__init__()
        self.layers = nn.Sequential(
            nn.Linear(in_dim, 1024), nn.Dropout(0.2), nn.Linear(1024, 128), nn.Dropout(0.2),
            nn.Linear(128, 64), nn.Dropout(0.1), nn.Linear(64, 16), nn.Linear(16, 1))

    def forward(self, x):
        return self.layers(x)


class AestheticReward(RewardFunction):
    frame_fractions = (0.25, 0.5, 0.75)

    def __init__(self, device: str = "cuda", model_name: str = "openai/clip-vit-large-patch14",
                 random_init: bool = False, mlp_path: str | None = None) -> None:
        self._device = device
        self.model_name, self.random_init, self.mlp_path = model_name, random_init, mlp_path
        self._tower = None
        self._mlp: AestheticMLP | None = None

    def _ensure_loaded(self) -> None:
        if self._tower is not None:
            return
        self._tower = build_image_tower(self.model_name, self._device, random_init=self.random_init)
        width = self._tower.proj.out_features
        mlp = AestheticMLP(width)
        if self.mlp_path:
            mlp.load_state_dict(torch.load(self.mlp_path, map_location="cpu"))
        else:
            gen = torch.Generator().manual_seed(1234)
            with torch.no_grad():
                for p in mlp.parameters():
                    if p.dim() > 1:
                        p.copy_(torch.randn(p.shape, generator=gen) / p.shape[1] ** 0.5)
        self._mlp = mlp.to(self._device).eval().requires_grad_(False)

    @torch.no_grad()
    def score_tensor_batch(self, outputs: torch.Tensor, prompts=None, metadata=None) -> torch.Tensor:
        self._ensure_loaded()
        frames = frames_for_scoring(outputs.to(self._device), self.frame_fractions)
        b, k = frames.shape[:2]
        feats = self._tower.features(frames.reshape(b * k, *frames.shape[2:]))
        return self._mlp(feats.float()).view(b, k).mean(dim=1)

    async def score(self, rollout: Rollout) -> float:
        return float(self.score_tensor_batch(rollout.trajectory.output.unsqueeze(0))[0])

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        outs = torch.stack([r.trajectory.output for r in rollouts])
        return self.score_tensor_batch(outs).tolist()
