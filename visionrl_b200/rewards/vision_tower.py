"""Image towers behind the model-backed rewards.

``build_image_tower(name)`` returns a :class:`ViTScorer`.  Names of the form
``random:<preset>[:seed]`` (or any name when ``random_init=True``) build the preset with
seeded random weights — the configuration used with synthetic data; a local directory with
``tower.safetensors`` in the native key layout, or with the files of a Hugging Face CLIP
checkpoint, is loaded instead.  Hub names cannot be resolved offline and raise with that
explanation.
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


def _local_tower(directory: str) -> ViTScorer:
    """A tower from a local directory: ``tower.safetensors`` in the native key layout, or the files
    of a Hugging Face CLIP checkpoint (``*.safetensors`` + ``config.json``), converted on the fly.
    Width, depth, patch and image size are read off the weights; the head count and the
    activation come from ``config.json`` (``vision_config`` of a two-tower config), defaulting to
    64-wide heads and the OpenAI ``quick_gelu``."""
    import json

    from safetensors.torch import load_file

    from visionrl_b200.models import convert

    native_file = os.path.join(directory, "tower.safetensors")
    if os.path.exists(native_file):
        state = load_file(native_file)
    else:
        files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors")) \
            if os.path.isdir(directory) else []
        if not files:
            raise FileNotFoundError(
                f"reward tower {directory!r}: no local tower.safetensors or Hugging Face *.safetensors; "
                "pass reward.kwargs.<name>.random_init=true (or model_name='random:vit_l14') for "
                "seeded random weights")
        raw: dict = {}
        for name in files:
            raw.update(load_file(os.path.join(directory, name)))
        state = convert.clip_vision_from_hf(raw)
    shape = convert.clip_vision_shape(state)
    heads, act = max(1, shape["dim"] // 64), "quick_gelu"
    config_file = os.path.join(directory, "config.json")
    if os.path.exists(config_file):
        with open(config_file) as fh:
            config = json.load(fh)
        vision = config.get("vision_config", config)
        heads = int(vision.get("num_attention_heads", heads))
        act = {"quick_gelu": "quick_gelu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh",
               "gelu_tanh": "gelu_tanh"}.get(str(vision.get("hidden_act", act)), act)
    tower = ViTScorer(heads=heads, act=act, **shape)
    result = tower.load_state_dict(state, strict=False)
    allowed = ("score_head.", "mean", "std")
    bad = [k for k in result.missing_keys if not k.startswith(allowed)] + list(result.unexpected_keys)
    if bad:
        raise ValueError(f"reward tower {directory!r}: keys that do not fit the tower: {bad[:4]}")
    return tower


def build_text_tower(directory: str, device: Any, dtype: Any = None):
    """``(CLIPTextTower, tokenizer, logit_scale)`` from a local Hugging Face CLIP checkpoint
    directory, or ``None`` when the directory does not hold a text tower and tokenizer files
    (``vocab.json`` + ``merges.txt``, read by ``transformers.CLIPTokenizer``)."""
    import json
    import math

    from safetensors.torch import load_file

    from visionrl_b200.models import convert
    from visionrl_b200.models.nn.vision import CLIPTextTower

    if not os.path.isdir(directory):
        return None
    if not all(os.path.exists(os.path.join(directory, f)) for f in ("vocab.json", "merges.txt")):
        return None
    raw: dict = {}
    for name in sorted(f for f in os.listdir(directory) if f.endswith(".safetensors") and f != "tower.safetensors"):
        raw.update(load_file(os.path.join(directory, name)))
    try:
        state = convert.clip_text_from_hf(raw)
    except KeyError:
        return None
    shape = convert.clip_text_shape(state)
    heads, act, eos = max(1, shape["dim"] // 64), "quick_gelu", None
    config_file = os.path.join(directory, "config.json")
    if os.path.exists(config_file):
        with open(config_file) as fh:
            config = json.load(fh)
        text = config.get("text_config", config)
        heads = int(text.get("num_attention_heads", heads))
        act = {"quick_gelu": "quick_gelu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh",
               "gelu_tanh": "gelu_tanh"}.get(str(text.get("hidden_act", act)), act)
        eos_id = text.get("eos_token_id")
        eos = None if eos_id in (None, 2) else int(eos_id)      # 2: the legacy configs, meaning "largest id"
    from transformers import CLIPTokenizer

    tokenizer = CLIPTokenizer.from_pretrained(directory)
    device = torch.device(device)
    dtype = tower_dtype(dtype, device)
    tower = CLIPTextTower(heads=heads, act=act, eos_token_id=eos, **shape)
    tower.load_state_dict(state, strict=True)
    scale = float(math.exp(float(raw["logit_scale"]))) if "logit_scale" in raw else 100.0
    return tower.to(device=device, dtype=dtype).eval().requires_grad_(False), tokenizer, scale


def tower_dtype(dtype: Any, device: torch.device) -> torch.dtype:
    """``None`` → bf16 on a GPU, fp32 on the host; otherwise a ``torch.dtype`` or its name
    (``"float32"``, ``"bfloat16"``, ``"bf16"``, ``"float16"``, ``"fp16"``)."""
    if dtype is None:
        return torch.bfloat16 if device.type == "cuda" else torch.float32
    if isinstance(dtype, torch.dtype):
        return dtype
    names = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
             "float16": torch.float16, "fp16": torch.float16, "half": torch.float16}
    key = str(dtype).replace("torch.", "").lower()
    if key not in names:
        raise ValueError(f"unknown reward tower dtype {dtype!r}")
    return names[key]


def build_image_tower(model_name: str, device: Any, dtype: Any = None,
                      random_init: bool = False) -> ViTScorer:
    device = torch.device(device)
    dtype = tower_dtype(dtype, device)
    seed = 0
    if model_name.startswith("random:"):
        parts = model_name.split(":")
        preset = parts[1]
        seed = int(parts[2]) if len(parts) > 2 else 0
        random_init = True
    else:
        preset = _PRESET_OF.get(model_name, "vit_l14")
    if random_init:
        # construction seeded too: every rank and every process scores with the same tower
        with seeded_construction(seed + 7919):
            tower = ViTScorer.from_preset(preset)
            seeded_init(tower, seed + 7919)
    else:
        with seeded_construction(seed + 7919):        # the scalar head is not part of a checkpoint
            tower = _local_tower(model_name)
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
