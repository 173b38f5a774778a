"""Image towers behind the model-backed rewards.

``build_image_tower(name)`` returns a :class:`ViTScorer`.  Names of the form
``random:<preset>[:seed]`` (or any name when ``random_init=True``) build the preset with
seeded random weights — the configuration used with synthetic data; a local directory
containing ``tower.safetensors`` in the native key layout is loaded instead.  Hub names
cannot be resolved offline and raise with that explanation.
"""

from __future__ import annotations

import os
from typing import Any

import torch

from visionrl_b200.models.families.flow_policy import seeded_construction, seeded_init
from visionrl_b200.models.nn.vision import ViTScorer

_PRESET_OF = {
    "openai/clip-vit-large-patch14": "vit_l14",
    "yuvalkirstain/PickScore_v1": "vit_l14",
    "laion/CLIP-ViT-H-14-laion2B-s32B-b79K": "vit_l14",
}


def build_image_tower(model_name: str, device: Any, dtype: torch.dtype | None = None,
                      random_init: bool = False) -> ViTScorer:
    device = torch.device(device)
    if dtype is None:
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    seed = 0
    if model_name.startswith("random:"):
        parts = model_name.split(":")
        preset = parts[1]
        seed = int(parts[2]) if len(parts) > 2 else 0
        random_init = True
    else:
        preset = _PRESET_OF.get(model_name, "vit_l14")
    # construction seeded too: every rank and every process scores with the same tower
    with seeded_construction(seed + 7919):
        tower = ViTScorer.from_preset(preset)
        if random_init:
            seeded_init(tower, seed + 7919)
    if not random_init:
        file = os.path.join(model_name, "tower.safetensors")
        if not os.path.exists(file):
            raise FileNotFoundError(
                f"reward tower {model_name!r}: no local {file}; pass reward.kwargs.<name>."
                "random_init=true (or model_name='random:vit_l14') for seeded random weights")
        from safetensors.torch import load_file

        tower.load_state_dict(load_file(file), strict=True)
    return tower.to(device=device, dtype=dtype).eval().requires_grad_(False)


def frames_for_scoring(output: torch.Tensor, fractions=(0.5,)) -> torch.Tensor:
    """``[B,3,H,W]`` images or ``[B,3,T,H,W]`` videos → ``[B, K, 3, H, W]`` sampled frames."""
    if output.ndim == 4:
        return output.unsqueeze(1)
    if output.ndim != 5:
        raise ValueError(f"expected [B,3,H,W] or [B,3,T,H,W], got {tuple(output.shape)}")
    t = output.shape[2]
    idx = [min(t - 1, max(0, int(t * f))) for f in fractions]
    return output[:, :, idx].permute(0, 2, 1, 3, 4)
