"""Aesthetic predictor: L2-normalised ViT-L/14 image features → MLP
``768→1024→128→64→16→1``; videos average the frames at 25/50/75 %
(reference: ``vrl/rewards/aesthetic.py:15-121``).

The MLP head is the public LAION "improved aesthetic predictor" (``sac+logos+ava1-l14-linearMSE.pth``,
3.7 MB, keys ``layers.{0,2,4,6,7}.{weight,bias}``).  The file is a third-party trained artefact and
is not redistributed with this package; it is looked up, in this order, at ``mlp_path``
(``reward.kwargs.aesthetic.mlp_path``), at ``$VRL_AESTHETIC_MLP`` and at
``visionrl_b200/rewards/assets/sac+logos+ava1-l14-linearMSE.pth`` (drop the file there to use it).
Without it — and always under ``random_init`` — a fixed-seed stand-in of the same shape is used,
which keeps the reward a deterministic function of the image for tests and benchmarks.
"""

from __future__ import annotations

import os
from pathlib import Path

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


ASSET_NAME = "sac+logos+ava1-l14-linearMSE.pth"


def resolve_mlp_weights(explicit: str | None = None) -> Path | None:
    """Path of the aesthetic head's weights, or ``None`` when no copy is available."""
    candidates = [explicit, os.environ.get("VRL_AESTHETIC_MLP"),
                  str(Path(__file__).with_name("assets") / ASSET_NAME)]
    for c in candidates:
        if c and Path(c).is_file():
            return Path(c)
    if explicit:
        raise FileNotFoundError(f"aesthetic MLP weights not found at {explicit}")
    return None


class AestheticReward(RewardFunction):
    frame_fractions = (0.25, 0.5, 0.75)

    def __init__(self, device: str = "cuda", dtype: str | None = None,
                 model_name: str = "openai/clip-vit-large-patch14",
                 random_init: bool = False, mlp_path: str | None = None) -> None:
        # positional order of the reference: (device, dtype, model_name); dtype None = bf16 on a GPU
        self._device, self._dtype = device, dtype
        self.model_name, self.random_init, self.mlp_path = model_name, random_init, mlp_path
        self._tower = None
        self._mlp: AestheticMLP | None = None

    def _ensure_loaded(self) -> None:
        if self._tower is not None:
            return
        self._tower = build_image_tower(self.model_name, self._device, self._dtype, random_init=self.random_init)
        width = self._tower.proj.out_features
        mlp = AestheticMLP(width)
        weights = None if self.random_init else resolve_mlp_weights(self.mlp_path)
        if weights is not None:
            mlp.load_state_dict(torch.load(weights, map_location="cpu"))
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
