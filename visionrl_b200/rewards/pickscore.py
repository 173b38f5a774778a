"""PickScore reward: ``logit_scale * <text, image> / 26`` on a CLIP-style tower
(reference: ``vrl/rewards/pickscore.py:15-100``)."""

from __future__ import annotations

from visionrl_b200.rewards.clip import CLIPScoreReward


class PickScoreReward(CLIPScoreReward):
    logit_scale = 100.0
    divisor = 26.0

    def __init__(self, device: str = "cuda", dtype: str | None = None,
                 processor_name: str = "laion/CLIP-ViT-H-14-laion2B-s32B-b79K",
                 model_name: str = "yuvalkirstain/PickScore_v1", random_init: bool = False) -> None:
        super().__init__(device=device, dtype=dtype, model_name=model_name, random_init=random_init)
        self.processor_name = processor_name
