"""Offline Diffusion-DPO trainer over preference pairs.

One ``step``: stack winner-then-loser pixels → latents and text conditioning (no
grad) → one noise draw and one timestep *per pair*, shared by winner and loser →
noised latents and regression target (``epsilon``: noise; ``v_prediction``: scheduler
velocity; ``flow_matching``: ``noise - latents`` with ``x_t = (1-sigma) x_0 + sigma noise``)
→ policy forward (grad) and reference forward (separate frozen model, or the policy
with adapters disabled) → DPO loss (+ ``sft_weight`` · MSE on the winner half) →
accumulate, clip, step.  A timestep *index* ``i`` is sampled and the model sees
``t = timesteps[i]`` with ``sigma = sigmas[i]``.  An empty or missing
``scheduler.timesteps`` is an error unless ``timestep_subset`` is given
(behavioural reference: ``vrl/trainers/offline_dpo.py:31-419``).
"""

from __future__ import annotations

import contextlib
import logging
from collections.abc import Callable, Iterable
from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from visionrl_b200.algorithms.dpo import diffusion_dpo_loss, diffusion_sft_loss
from visionrl_b200.trainers.base import raise_on_kernel_timeout

logger = logging.getLogger(__name__)


@dataclass(slots=True)
class OfflineDPOTrainerConfig:
    beta: float = 5000.0
    sft_weight: float = 0.0
    lr: float = 1e-8
    scale_lr: bool = True
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_weight_decay: float = 1e-2
    adam_epsilon: float = 1e-8
    use_adafactor: bool = False
    max_grad_norm: float = 1.0
    gradient_accumulation_steps: int = 1
    prediction_type: str = "flow_matching"
    num_train_timesteps: int = 1000
    timestep_subset: tuple[int, int] | None = None
    num_frames: int = 1
    vae_scale_factor_temporal: int = 1
    mixed_precision: str = "bf16"
    log_every: int = 10


@dataclass(slots=True)
class DPOStepMetrics:
    loss: float = 0.0
    raw_model_loss: float = 0.0
    raw_ref_loss: float = 0.0
    model_diff: float = 0.0
    ref_diff: float = 0.0
    implicit_acc: float = 0.0
    sft_loss: float = 0.0
    grad_norm: float = 0.0


ForwardFn = Callable[..., torch.Tensor]


def _backbone(model: nn.Module) -> nn.Module:
    inner = getattr(model, "transformer", None)
    return inner if inner is not None else model


def wan_forward(model, noisy_latents, timesteps, encoder_hidden_states, extra=None):
    """Video-DiT forward; a policy wrapper is unwrapped to its ``transformer`` first.  Native
    backbones take ``(latents, timestep, context)``; keyword-style backbones get the
    ``hidden_states=/timestep=/encoder_hidden_states=`` call and a tuple return."""
    del extra
    net = _backbone(model)
    if getattr(net, "cfg", None) is not None and hasattr(net, "patchify"):
        return net(noisy_latents, timesteps, encoder_hidden_states)
    return net(hidden_states=noisy_latents, timestep=timesteps,
               encoder_hidden_states=encoder_hidden_states, return_dict=False)[0]


def sd_unet_forward(model, noisy_latents, timesteps, encoder_hidden_states, extra=None):
    return model(sample=noisy_latents, timestep=timesteps,
                 encoder_hidden_states=encoder_hidden_states,
                 added_cond_kwargs=(extra or {}).get("added_cond_kwargs"), return_dict=False)[0]


def _build_optimizer(parameters: Iterable[nn.Parameter], cfg: OfflineDPOTrainerConfig):
    params = list(parameters)
    if cfg.use_adafactor:
        from transformers.optimization import Adafactor

        return Adafactor(params, lr=cfg.lr, scale_parameter=False, relative_step=False,
                         warmup_init=False, weight_decay=cfg.adam_weight_decay)
    from visionrl_b200.ops.optim import FusedAdamW

    return FusedAdamW(params, lr=cfg.lr, betas=(cfg.adam_beta1, cfg.adam_beta2),
                      weight_decay=cfg.adam_weight_decay, eps=cfg.adam_epsilon)


class OfflineDPOTrainer:
    def __init__(self, model: nn.Module, ref_model: nn.Module | None, forward_fn: ForwardFn,
                 noise_scheduler: Any, encode_pixels: Callable[[torch.Tensor], torch.Tensor],
                 encode_text: Callable[[list[str]], torch.Tensor],
                 config: OfflineDPOTrainerConfig | None = None,
                 device: torch.device | str = "cuda", grad_sync: Any | None = None) -> None:
        self.model, self.ref_model, self.forward_fn = model, ref_model, forward_fn
        self.noise_scheduler = noise_scheduler
        self.encode_pixels, self.encode_text = encode_pixels, encode_text
        self.config = config or OfflineDPOTrainerConfig()
        self.device = torch.device(device) if isinstance(device, str) else device
        self.global_step = 0
        self.grad_sync = grad_sync
        if self.ref_model is not None:
            self.ref_model.eval()
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
        trainable = [p for p in model.parameters() if p.requires_grad]
        if not trainable:
            raise RuntimeError("model has no trainable parameters — wire up LoRA / unfreeze first")
        self._optimizer = _build_optimizer(trainable, self.config)

    def _sample_timesteps(self, bsz: int) -> torch.Tensor:
        if self.config.timestep_subset is not None:
            lo, hi = self.config.timestep_subset
        else:
            ts = getattr(self.noise_scheduler, "timesteps", None)
            if ts is None or len(ts) == 0:
                raise RuntimeError(
                    "noise_scheduler.timesteps is empty/missing. Call "
                    "scheduler.set_timesteps(n) before training or pass "
                    "OfflineDPOTrainerConfig.timestep_subset=(lo, hi).")
            lo, hi = 0, len(ts)
        return torch.randint(lo, hi, (bsz,), device=self.device).long()

    def _timestep_values(self, index: torch.Tensor) -> torch.Tensor:
        ts = getattr(self.noise_scheduler, "timesteps", None)
        if ts is None or len(ts) == 0 or int(index.max()) >= len(ts):
            return index
        return ts.to(self.device)[index]

    def _inject_noise(self, latents, noise, index):
        """``index`` selects a schedule entry.  Returns ``(noisy, target, timestep_values)``."""
        kind = self.config.prediction_type
        sched = self.noise_scheduler
        if kind in ("epsilon", "v_prediction"):
            noisy = sched.add_noise(latents, noise, index)
            target = noise if kind == "epsilon" else sched.get_velocity(latents, noise, index)
            return noisy, target, index
        if kind != "flow_matching":
            raise ValueError(f"unknown prediction_type: {kind}")
        t_vals = self._timestep_values(index)
        sigmas = getattr(sched, "sigmas", None)
        if sigmas is not None and int(index.max()) < len(sigmas):
            sigma = sigmas.to(latents.device)[index].view(-1, *([1] * (latents.ndim - 1)))
            noisy = (1.0 - sigma) * latents + sigma * noise
        else:
            noisy = sched.scale_noise(latents, t_vals, noise)
        return noisy, noise - latents, t_vals

    def _autocast(self):
        kind = self.config.mixed_precision
        if self.device.type != "cuda" or kind not in ("fp16", "bf16"):
            return contextlib.nullcontext()
        first = next(iter(self.model.parameters()))
        if first.dtype != torch.float32:
            return contextlib.nullcontext()
        return torch.amp.autocast("cuda", dtype=torch.float16 if kind == "fp16" else torch.bfloat16)

    def _reference_forward(self, noisy, timesteps, ctx):
        if self.ref_model is not None:
            return self.forward_fn(self.ref_model, noisy, timesteps, ctx)
        if hasattr(self.model, "disable_adapter"):
            with self.model.disable_adapter():
                return self.forward_fn(self.model, noisy, timesteps, ctx)
        raise RuntimeError("no ref_model and policy has no ``disable_adapter`` — cannot compute "
                           "reference prediction")

    def step(self, batch: Any) -> DPOStepMetrics:
        cfg = self.config
        self.model.train()
        with torch.no_grad():
            latents = batch.latents_winner_then_loser().to(self.device) \
                if hasattr(batch, "latents_winner_then_loser") \
                else self.encode_pixels(batch.stacked_winner_then_loser().to(self.device))
            ctx = self.encode_text(batch.captions)
            if ctx.shape[0] != latents.shape[0]:
                ctx = ctx.repeat(latents.shape[0] // ctx.shape[0], *([1] * (ctx.ndim - 1)))
        pairs = latents.shape[0] // 2
        tile = (2, *([1] * (latents.ndim - 1)))
        noise = torch.randn((pairs, *latents.shape[1:]), device=latents.device,
                            dtype=latents.dtype).repeat(*tile)
        index = self._sample_timesteps(pairs).repeat(2)
        noisy, target, t_vals = self._inject_noise(latents, noise, index)
        with self._autocast():
            pred = self.forward_fn(self.model, noisy, t_vals, ctx)
            with torch.no_grad():
                ref = self._reference_forward(noisy, t_vals, ctx).detach()
            stats = diffusion_dpo_loss(pred.float(), ref.float(), target.float(), cfg.beta)
            loss = stats["loss"]
            sft = torch.zeros((), device=self.device)
            if cfg.sft_weight > 0:
                sft = diffusion_sft_loss(pred[:pairs].float(), target[:pairs].float())
                loss = loss + cfg.sft_weight * sft
        (loss / max(1, cfg.gradient_accumulation_steps)).backward()
        grad_norm: Any = 0.0
        if (self.global_step + 1) % cfg.gradient_accumulation_steps == 0:
            if self.grad_sync is not None:
                grad_norm = self.grad_sync.reduce_clip_step(self._optimizer, cfg.max_grad_norm)
            elif callable(getattr(self._optimizer, "grad_norm", None)):
                grad_norm = self._optimizer.grad_norm()
                coef = (cfg.max_grad_norm / (grad_norm + 1e-6)).clamp(max=1.0) \
                    if cfg.max_grad_norm > 0 else None
                self._optimizer.step(clip_coef=coef)
            else:
                if cfg.max_grad_norm > 0:
                    grad_norm = nn.utils.clip_grad_norm_(self.model.parameters(), cfg.max_grad_norm)
                self._optimizer.step()
            self._optimizer.zero_grad()
        self.global_step += 1
        raise_on_kernel_timeout(self.device, self.grad_sync, f"DPO step {self.global_step}")
        vals = torch.stack([stats[k].detach().float() for k in
                            ("loss", "raw_model_loss", "raw_ref_loss", "model_diff", "ref_diff",
                             "implicit_acc")] + [sft.detach().float(),
                            torch.as_tensor(grad_norm, dtype=torch.float32, device=sft.device).reshape(())]).tolist()
        return DPOStepMetrics(*vals)

    def state_dict(self) -> dict[str, Any]:
        return {"global_step": self.global_step, "optimizer": self._optimizer.state_dict()}

    def load_state_dict(self, state: dict[str, Any], *, strict: bool = True) -> None:
        if not isinstance(state, dict):
            raise TypeError("OfflineDPOTrainer.load_state_dict expects a dict")
        self.global_step = int(state.get("global_step", state.get("step", 0)))
        if "optimizer" in state:
            try:
                self._optimizer.load_state_dict(state["optimizer"])
            except Exception:
                if strict:
                    raise
                logger.warning("Skipping incompatible optimizer state during non-strict load")
        elif strict:
            raise ValueError("checkpoint missing optimizer state")


__all__ = ["DPOStepMetrics", "ForwardFn", "OfflineDPOTrainer", "OfflineDPOTrainerConfig",
           "sd_unet_forward", "wan_forward"]
