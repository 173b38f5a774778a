"""CLIP-score reward: image/text cosine similarity × logit scale / 30; videos use the middle
frame (reference: ``vrl/rewards/clip.py:15-103``).  With ``model_name`` a local Hugging Face CLIP
checkpoint directory (weights, ``config.json``, ``vocab.json``, ``merges.txt``) both towers and the
logit scale come from it; otherwise the text side is a seeded embedding of the prompt in the
image tower's feature space."""

from __future__ import annotations

import torch

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.models.nn.vision import SyntheticTextEncoder
from visionrl_b200.rewards.base import RewardFunction
from visionrl_b200.rewards.vision_tower import build_image_tower, build_text_tower, frames_for_scoring


class CLIPScoreReward(RewardFunction):
    logit_scale = 100.0
    divisor = 30.0

    def __init__(self, device: str = "cuda", model_name: str = "openai/clip-vit-large-patch14",
                 random_init: bool = False, dtype: str | None = None) -> None:
        self._device, self._dtype = device, dtype
        self.model_name, self.random_init = model_name, random_init
        self._tower = None
        self._text: SyntheticTextEncoder | None = None

    def _ensure_loaded(self) -> None:
        if self._tower is None:
            self._tower = build_image_tower(self.model_name, self._device, self._dtype,
                                            random_init=self.random_init)
            self._text = SyntheticTextEncoder(self._tower.proj.out_features, 0, salt="clip-text")
            self._text_tower = None
            if not self.random_init and not self.model_name.startswith("random:"):
                # a local checkpoint directory with its text tower and tokenizer files scores
                # prompts with the real text side and the checkpoint's own logit scale
                real = build_text_tower(self.model_name, self._device, self._dtype)
                if real is not None:
                    self._text_tower, self._tokenizer, self.logit_scale = real

    def _text_features(self, prompts: list[str]) -> torch.Tensor:
        if getattr(self, "_text_tower", None) is not None:
            tower = self._text_tower
            ids = self._tokenizer(list(prompts), padding="max_length", truncation=True,
                                  max_length=tower.context, return_tensors="pt")["input_ids"]
            return tower.features(ids.to(self._device))
        emb, _ = self._text(prompts, 1, self._device, torch.float32)
        emb = emb[:, 0]
        return emb / emb.norm(dim=-1, keepdim=True).clamp_min(1e-6)

    @torch.no_grad()
    def score_tensor_batch(self, outputs: torch.Tensor, prompts, metadata=None) -> torch.Tensor:
        self._ensure_loaded()
        frames = frames_for_scoring(outputs.to(self._device), (0.5,))[:, 0]
        img = self._tower.features(frames)
        return self.logit_scale * (img * self._text_features(list(prompts))).sum(-1) / self.divisor

    async def score(self, rollout: Rollout) -> float:
        return float(self.score_tensor_batch(rollout.trajectory.output.unsqueeze(0),
                                             [rollout.trajectory.prompt])[0])

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        outs = torch.stack([r.trajectory.output for r in rollouts])
        return self.score_tensor_batch(outs, [r.trajectory.prompt for r in rollouts]).tolist()
