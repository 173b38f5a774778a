"""SD3.5 family: MMDiT transformer + 16-channel image latent decoder
(reference adapter: ``vrl/models/families/sd3_5/policy.py:57-389``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.models.families.flow_policy import FlowSamplingState, NativeFlowPolicy
from visionrl_b200.models.nn.mmdit import MMDiT, MMDiTConfig
from visionrl_b200.models.nn.vision import LatentDecoder2D, SyntheticTextEncoder

SD3SamplingState = FlowSamplingState


class SD3_5Policy(NativeFlowPolicy):
    family = "sd3_5"
    latent_rank = 4
    default_shift = 3.0
    context_length = 154

    @classmethod
    def _build_modules(cls, arch: dict[str, Any], native: dict[str, Any]):
        cfg = MMDiTConfig.from_dict(arch)
        transformer = MMDiT(cfg)
        dec = dict(native.get("decoder") or {})
        decoder = None
        if dec.get("enable", True):
            decoder = LatentDecoder2D(cfg.in_channels, int(dec.get("base", 128)),
                                      tuple(dec.get("mults", (1, 2, 4, 4))),
                                      int(dec.get("blocks", 2)))
        return transformer, decoder, SyntheticTextEncoder(cfg.context_dim, cfg.pooled_dim)

    @classmethod
    def _build_prompt_encoder(cls, path: str, arch: dict[str, Any], device):
        from visionrl_b200.models.nn.prompt_encoders import SD3PromptEncoder

        cfg = MMDiTConfig.from_dict(arch)
        encoder = SD3PromptEncoder.from_directory(path, cfg.context_dim, device)
        if encoder.pooled_dim != cfg.pooled_dim:
            raise ValueError(f"the CLIP towers pool to {encoder.pooled_dim} values, the transformer expects "
                             f"{cfg.pooled_dim} (model.arch.pooled_dim)")
        return encoder

    def _context_tokens(self, max_sequence_length: int) -> int:
        # two 77-token CLIP segments are concatenated in front of the T5 tokens; a
        # fixed ``context_len`` in the arch overrides it (tiny models)
        fixed = self.arch.get("context_len")
        if fixed:
            return int(fixed)
        from visionrl_b200.models.nn.prompt_encoders import CLIP_TOKENS, SD3PromptEncoder

        if isinstance(self._frozen.text, SD3PromptEncoder):
            # the public pipeline's meaning: CLIP tokens first, then max_sequence_length T5 tokens
            return CLIP_TOKENS + max_sequence_length
        return max_sequence_length

    def _call_transformer(self, latents, timesteps, embeds, pooled, state):
        return self.transformer(latents, timesteps, embeds, pooled)


__all__ = ["SD3SamplingState", "SD3_5Policy"]
