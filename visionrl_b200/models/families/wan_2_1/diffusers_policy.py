"""Wan-2.1 text-to-video family: video DiT with 3-D RoPE and cross-attention to text tokens,
5-D latents ``[B, C, T, H, W]``, batched CFG, per-channel latent de-normalisation before the
frame decoder (reference adapter: ``vrl/models/families/wan_2_1/diffusers_policy.py:50-363``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.models.families.flow_policy import FlowSamplingState, NativeFlowPolicy
from visionrl_b200.models.nn.vision import LatentDecoder3D, SyntheticTextEncoder
from visionrl_b200.models.nn.wan import WanConfig, WanDiT

WanSamplingState = FlowSamplingState


class WanT2VDiffusersPolicy(NativeFlowPolicy):
    family = "wan_2_1"
    latent_rank = 5
    default_shift = 3.0
    context_length = 512

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self.sequence_parallel = None     # set by parallel.ulysses.attach_sequence_parallel

    @classmethod
    def _build_prompt_encoder(cls, path: str, arch: dict[str, Any], device):
        from visionrl_b200.models.nn.prompt_encoders import UMT5PromptEncoder

        encoder = UMT5PromptEncoder.from_directory(path, device)
        width = int(WanConfig.from_dict(arch).text_dim)
        if encoder.context_dim != width:
            raise ValueError(f"the text encoder is {encoder.context_dim} wide, the transformer expects "
                             f"{width} (model.arch.text_dim)")
        return encoder

    @classmethod
    def _build_modules(cls, arch: dict[str, Any], native: dict[str, Any]):
        cfg = WanConfig.from_dict(arch)
        dec = dict(native.get("decoder") or {})
        decoder = None
        if dec.get("enable", True):
            decoder = LatentDecoder3D(cfg.out_channels, int(dec.get("base", 96)),
                                      tuple(dec.get("mults", (1, 2, 4, 4))),
                                      int(dec.get("blocks", 2)),
                                      int(arch.get("vae_temporal_scale", 4)))
        return WanDiT(cfg), decoder, SyntheticTextEncoder(cfg.text_dim, 0)

    def _context_tokens(self, max_sequence_length: int) -> int:
        fixed = self.arch.get("context_len")
        return int(fixed) if fixed else max_sequence_length

    def _call_transformer(self, latents, timesteps, embeds, pooled, state):
        return self.transformer(latents, timesteps, embeds, sp=self.sequence_parallel)


WanT2VSamplingState = WanSamplingState

__all__ = ["WanSamplingState", "WanT2VDiffusersPolicy", "WanT2VSamplingState"]
