"""Prompt conditioning from real text encoders, behind the interface of the synthetic one.

``SyntheticTextEncoder`` (seeded embeddings) is what the policies use when no checkpoint is
around.  The classes here compute the same ``(context, pooled)`` pair with the native CLIP text
tower and T5 / UMT5 encoder from a local checkpoint directory in the pipeline layout
(``text_encoder*/`` with ``*.safetensors`` + ``config.json``, ``tokenizer*/``), following what the
public pipelines do:

* Wan / Cosmos (``UMT5PromptEncoder``): the prompt is tokenised to ``length`` tokens, encoded
  with the attention mask, and everything after the prompt's own tokens is set to zero;
* SD3.5 (``SD3PromptEncoder``): two CLIP towers give their second-to-last hidden states for 77
  tokens, concatenated on the feature axis and zero-padded to the T5 width, and their projected
  end-of-text states concatenated as the pooled vector; T5 encodes ``length - 77`` tokens
  (without a mask); the context is the CLIP part followed by the T5 part.

Results are cached per prompt in (pinned) host memory and copied to the device on demand by the
base class, so a training step moves the same bytes whichever encoder produced them.
"""

from __future__ import annotations

import json
import os
from typing import Any

import torch

from visionrl_b200.models import convert
from visionrl_b200.models.nn.text_encoders import T5Encoder, T5EncoderConfig
from visionrl_b200.models.nn.vision import CLIPTextTower, SyntheticTextEncoder

CLIP_TOKENS = 77


def _read_dir(directory: str) -> tuple[dict[str, torch.Tensor], dict]:
    from safetensors.torch import load_file

    if not os.path.isdir(directory):
        raise FileNotFoundError(f"text encoder directory not found: {directory}")
    state: dict[str, torch.Tensor] = {}
    for name in sorted(f for f in os.listdir(directory) if f.endswith(".safetensors")):
        state.update(load_file(os.path.join(directory, name)))
    if not state:
        raise FileNotFoundError(f"no .safetensors files in {directory}")
    config_file = os.path.join(directory, "config.json")
    config = json.load(open(config_file)) if os.path.exists(config_file) else {}
    return state, config


def load_t5_encoder(directory: str) -> T5Encoder:
    state, config = _read_dir(directory)
    if not config:
        raise FileNotFoundError(f"{directory}/config.json is needed to size the T5 encoder")
    encoder = T5Encoder(T5EncoderConfig.from_hf(config))
    encoder.load_state_dict(convert.t5_encoder_from_hf(state), strict=True)
    return encoder.eval().requires_grad_(False)


def load_clip_text_tower(directory: str) -> CLIPTextTower:
    state, config = _read_dir(directory)
    native = convert.clip_text_from_hf(state)
    shape = convert.clip_text_shape(native)
    text = config.get("text_config", config)
    heads = int(text.get("num_attention_heads", max(1, shape["dim"] // 64)))
    act = {"quick_gelu": "quick_gelu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh"}.get(
        str(text.get("hidden_act", "quick_gelu")), "quick_gelu")
    eos = text.get("eos_token_id")
    tower = CLIPTextTower(heads=heads, act=act, eos_token_id=None if eos in (None, 2) else int(eos), **shape)
    tower.load_state_dict(native, strict=True)
    return tower.eval().requires_grad_(False)


def load_tokenizer(directory: str) -> Any:
    """The tokenizer a checkpoint directory describes; a directory with nothing but ``vocab.json``
    and ``merges.txt`` is read as a CLIP byte-pair vocabulary."""
    from transformers import AutoTokenizer, CLIPTokenizer

    names = set(os.listdir(directory)) if os.path.isdir(directory) else set()
    if {"vocab.json", "merges.txt"} <= names and not names & {"tokenizer.json", "tokenizer_config.json"}:
        return CLIPTokenizer.from_pretrained(directory)
    return AutoTokenizer.from_pretrained(directory)


class _EncodedPromptCache(SyntheticTextEncoder):
    """The host/device caches and transfer accounting of the synthetic encoder around a real
    ``encode(prompt, length) -> (context[length, D], pooled[P])``."""

    def encode(self, prompt: str, length: int) -> tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def _host_entry(self, prompt: str, length: int, dtype):
        key = (prompt, length, dtype)
        if key not in self._host:
            with torch.no_grad():
                context, pooled = self.encode(prompt, length)
            context, pooled = context.to("cpu", dtype).contiguous(), pooled.to("cpu", dtype).contiguous()
            if torch.cuda.is_available():
                context, pooled = context.pin_memory(), pooled.pin_memory()
            self._host[key] = (context, pooled)
        return self._host[key]


class UMT5PromptEncoder(_EncodedPromptCache):
    def __init__(self, encoder: T5Encoder, tokenizer: Any, device: Any = "cpu"):
        super().__init__(encoder.cfg.d_model, 0, salt="umt5")
        self.encoder, self.tokenizer = encoder.to(device), tokenizer
        self.device = torch.device(device)

    @classmethod
    def from_directory(cls, path: str, device: Any = "cpu") -> "UMT5PromptEncoder":
        return cls(load_t5_encoder(os.path.join(path, "text_encoder")),
                   load_tokenizer(os.path.join(path, "tokenizer")), device)

    def encode(self, prompt: str, length: int):
        batch = self.tokenizer([prompt], padding="max_length", max_length=length, truncation=True,
                               add_special_tokens=True, return_attention_mask=True, return_tensors="pt")
        ids, mask = batch["input_ids"].to(self.device), batch["attention_mask"].to(self.device)
        hidden = self.encoder(ids, mask)[0].float()
        hidden = hidden * mask[0].unsqueeze(-1)                 # nothing after the prompt's own tokens
        return hidden, torch.zeros(1)


class SD3PromptEncoder(_EncodedPromptCache):
    def __init__(self, clip_l: CLIPTextTower, tok_l: Any, clip_g: CLIPTextTower, tok_g: Any,
                 t5: T5Encoder | None, tok_t5: Any, joint_dim: int, device: Any = "cpu"):
        pooled = clip_l.proj.out_features + clip_g.proj.out_features
        super().__init__(joint_dim, pooled, salt="sd3")
        self.device = torch.device(device)
        self.clip_l, self.clip_g = clip_l.to(device), clip_g.to(device)
        self.t5 = t5.to(device) if t5 is not None else None
        self.tok_l, self.tok_g, self.tok_t5 = tok_l, tok_g, tok_t5
        clip_width = clip_l.token_embed.embedding_dim + clip_g.token_embed.embedding_dim
        if clip_width > joint_dim:
            raise ValueError(f"the CLIP towers are {clip_width} wide together, the context only {joint_dim}")
        if t5 is not None and t5.cfg.d_model != joint_dim:
            raise ValueError(f"the T5 encoder is {t5.cfg.d_model} wide, the context {joint_dim}")

    @classmethod
    def from_directory(cls, path: str, joint_dim: int, device: Any = "cpu") -> "SD3PromptEncoder":
        """``text_encoder`` + ``tokenizer`` (CLIP-L), ``text_encoder_2`` + ``tokenizer_2`` (CLIP-G)
        and, when present, ``text_encoder_3`` + ``tokenizer_3`` (T5; without it that part of the
        context is zeros, as the public pipeline does)."""
        sub = lambda name: os.path.join(path, name)  # noqa: E731
        t5 = tok3 = None
        if os.path.isdir(sub("text_encoder_3")):
            t5, tok3 = load_t5_encoder(sub("text_encoder_3")), load_tokenizer(sub("tokenizer_3"))
        return cls(load_clip_text_tower(sub("text_encoder")), load_tokenizer(sub("tokenizer")),
                   load_clip_text_tower(sub("text_encoder_2")), load_tokenizer(sub("tokenizer_2")),
                   t5, tok3, joint_dim, device)

    def _clip(self, tower: CLIPTextTower, tokenizer: Any, prompt: str):
        ids = tokenizer([prompt], padding="max_length", max_length=min(CLIP_TOKENS, tower.context), truncation=True,
                        return_tensors="pt")["input_ids"].to(self.device)
        hidden, pooled = tower.encode(ids)
        return hidden[0].float(), pooled[0].float()

    def encode(self, prompt: str, length: int):
        h_l, p_l = self._clip(self.clip_l, self.tok_l, prompt)
        h_g, p_g = self._clip(self.clip_g, self.tok_g, prompt)
        clip = torch.cat([h_l, h_g], dim=-1)
        clip = torch.nn.functional.pad(clip, (0, self.context_dim - clip.shape[-1]))
        t5_len = length - clip.shape[0]
        if t5_len < 0:
            raise ValueError(f"a context of {length} tokens cannot hold the {clip.shape[0]} CLIP tokens")
        if self.t5 is None or t5_len == 0:
            tail = torch.zeros(t5_len, self.context_dim, device=clip.device)
        else:
            ids = self.tok_t5([prompt], padding="max_length", max_length=t5_len, truncation=True,
                              add_special_tokens=True, return_tensors="pt")["input_ids"].to(self.device)
            tail = self.t5(ids)[0].float()
        return torch.cat([clip, tail], dim=0), torch.cat([p_l, p_g], dim=-1)


__all__ = ["CLIP_TOKENS", "SD3PromptEncoder", "UMT5PromptEncoder", "load_clip_text_tower", "load_t5_encoder",
           "load_tokenizer"]
