"""Cosmos-Predict2-style video-to-world family.

The transformer sees ``[latents ⊙ (1-m) + cond ⊙ m ; m]`` (conditioning frames blended in by an
indicator mask that also enters as an extra channel) with EDM-style preconditioning
``t = sigma / (sigma + 1)``, ``c_in = c_skip = 1 - t``, ``c_out = -t``.  The denoised estimate of
both CFG branches is blended with the conditioning frames, guidance is
``cond + g * (cond - uncond)`` (two sequential forwards), and the velocity handed to the SDE
step is ``(latents - combined) / sigma``.  ``forward_step`` reads ``scheduler.sigmas[step_idx]``,
so the replay passes the true step index (reference:
``vrl/models/families/cosmos/policy.py:59-571``).
"""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.models.diffusion import VideoGenerationRequest
from visionrl_b200.models.families.flow_policy import FlowSamplingState, NativeFlowPolicy
from visionrl_b200.models.nn.vision import LatentDecoder3D, SyntheticTextEncoder
from visionrl_b200.models.nn.wan import WanConfig, WanDiT

CosmosSamplingState = FlowSamplingState


class CosmosPredict2Policy(NativeFlowPolicy):
    family = "cosmos"
    latent_rank = 5
    default_shift = 1.0
    context_length = 512
    num_cond_latent_frames = 1

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self.reference_image: Any = None
        self.sequence_parallel = None

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
        arch = dict(arch)
        arch["extra_in_channels"] = 1
        cfg = WanConfig.from_dict(arch)
        dec = dict(native.get("decoder") or {})
        decoder = None
        if dec.get("enable", True):
            decoder = LatentDecoder3D(cfg.out_channels, int(dec.get("base", 96)),
                                      tuple(dec.get("mults", (1, 2, 4, 4))),
                                      int(dec.get("blocks", 2)),
                                      int(arch.get("vae_temporal_scale", 4)))
        return WanDiT(cfg), decoder, SyntheticTextEncoder(cfg.text_dim, 0)

    def set_reference_image(self, image: Any) -> None:
        self.reference_image = image

    def _reference_latent(self, image: Any, shape: tuple, batch: int) -> torch.Tensor:
        """Conditioning latent frames: a seeded encoding of the reference image, zeros if none."""
        c, f, h, w = shape
        cond = torch.zeros(batch, c, f, h, w, device=self._device, dtype=torch.float32)
        if image is None or (isinstance(image, str) and not image):
            return cond
        if isinstance(image, torch.Tensor):
            img = image.float().to(self._device)
            if img.ndim == 3:
                img = img.unsqueeze(0)
            pooled = torch.nn.functional.adaptive_avg_pool2d(img, (h, w)).mean(1, keepdim=True)
            cond[:, :, : self.num_cond_latent_frames] = pooled.unsqueeze(2).expand(
                batch, c, self.num_cond_latent_frames, h, w)
            return cond
        import hashlib

        seed = int.from_bytes(hashlib.sha256(str(image).encode()).digest()[:8], "little") >> 1
        gen = torch.Generator().manual_seed(seed)
        frame = torch.randn(c, self.num_cond_latent_frames, h, w, generator=gen)
        cond[:, :, : self.num_cond_latent_frames] = frame.to(self._device)
        return cond

    def prepare_sampling(self, request: VideoGenerationRequest, encoded: dict[str, Any],
                         **kwargs: Any) -> FlowSamplingState:
        state = super().prepare_sampling(request, encoded)
        b = state.latents.shape[0]
        shape = tuple(state.latents.shape[1:])
        image = kwargs.get("reference_image", self.reference_image)
        indicator = torch.zeros(1, 1, shape[1], 1, 1, device=self._device)
        indicator[:, :, : self.num_cond_latent_frames] = 1.0
        state.extra = {
            "init_latents": self._reference_latent(image, shape, b),
            "cond_indicator": indicator, "uncond_indicator": indicator.clone(),
            "cond_mask": indicator.expand(1, 1, *shape[1:]).contiguous(),
            "uncond_mask": indicator.expand(1, 1, *shape[1:]).contiguous(),
            "padding_mask": torch.zeros(1, 1, shape[2], shape[3], device=self._device),
            "fps": int(getattr(request, "fps", 16)), "sigma_conditioning": 0.0001,
        }
        return state

    def _denoise(self, state: FlowSamplingState, sigma: torch.Tensor, embeds: torch.Tensor,
                 indicator: torch.Tensor) -> torch.Tensor:
        x = state.latents.float()
        init = state.extra["init_latents"]
        t = sigma / (sigma + 1)
        c_in, c_skip, c_out = 1 - t, 1 - t, -t
        blended = indicator * init + (1 - indicator) * (x * c_in)
        mask = indicator.expand(x.shape[0], 1, *x.shape[2:])
        net_in = torch.cat([blended, mask], dim=1)
        out = self.transformer(net_in, (t * 1000).expand(x.shape[0]), embeds,
                               sp=self.sequence_parallel).float()
        denoised = c_skip * x + c_out * out
        return indicator * init + (1 - indicator) * denoised

    def forward_step(self, state: FlowSamplingState, step_idx: int) -> dict[str, Any]:
        sigma = state.scheduler.sigmas.to(self._device)[step_idx].float().clamp_min(1e-5)
        cond = self._denoise(state, sigma, state.prompt_embeds, state.extra["cond_indicator"])
        if state.do_cfg:
            uncond = self._denoise(state, sigma, state.negative_prompt_embeds,
                                   state.extra["uncond_indicator"])
            combined = cond + state.guidance_scale * (cond - uncond)
        else:
            uncond, combined = torch.zeros_like(cond), cond
        noise_pred = (state.latents.float() - combined) / sigma
        return {"noise_pred": noise_pred, "noise_pred_cond": cond, "noise_pred_uncond": uncond}

    def export_batch_context(self, state: FlowSamplingState) -> dict[str, Any]:
        ctx = super().export_batch_context(state)
        for key in ("fps", "cond_mask", "uncond_mask", "padding_mask", "cond_indicator",
                    "uncond_indicator", "sigma_conditioning"):
            ctx[key] = state.extra[key]
        return ctx

    def export_training_extras(self, state: FlowSamplingState) -> dict[str, Any]:
        out = super().export_training_extras(state)
        out["init_latents"] = state.extra["init_latents"]
        return out

    def restore_eval_state(self, batch_extras, batch_context, latents, step_idx) -> FlowSamplingState:
        state = super().restore_eval_state(batch_extras, batch_context, latents, step_idx)
        state.scheduler = self._scheduler
        state.extra = {k: batch_context[k] for k in ("cond_indicator", "uncond_indicator", "fps")}
        state.extra["init_latents"] = batch_extras["init_latents"]
        return state

    def replay_forward(self, batch: Any, timestep_idx: int) -> dict[str, Any]:
        state = self.restore_eval_state(batch.extras, batch.context,
                                        batch.observations[:, timestep_idx], timestep_idx)
        return self.forward(state, timestep_idx)


CosmosPredict2SamplingState = CosmosSamplingState

__all__ = ["CosmosPredict2Policy", "CosmosPredict2SamplingState", "CosmosSamplingState"]
