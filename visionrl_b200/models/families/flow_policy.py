"""Native flow-matching diffusion policy shared by the SD3.5, Wan and Cosmos families.

The trainable transformer is the only registered child module, so
``state_dict()`` has ``transformer.*`` keys only; the frozen latent decoder and the
text conditioner are held outside the module tree.  Classifier-free guidance is
batched as ``[negative, positive]`` in one forward and combined as
``uncond + g * (cond - uncond)`` in fp32 (reference behaviour:
``vrl/models/families/sd3_5/policy.py:268-325``).  Initial latents are fp32 and
seeded per request.
"""

from __future__ import annotations

import contextlib
import math
import random
import sys
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Any

import torch
from torch import nn

from visionrl_b200.models.diffusion import DiffusionPolicy, VideoGenerationRequest
from visionrl_b200.models.nn.layers import apply_lora
from visionrl_b200.models.nn.scheduler import FlowMatchEulerScheduler


@dataclass
class FlowSamplingState:
    """Private sampling state; the engine reads only ``latents`` / ``timesteps`` / ``scheduler``."""

    latents: torch.Tensor
    timesteps: torch.Tensor
    scheduler: Any
    prompt_embeds: torch.Tensor
    pooled_prompt_embeds: torch.Tensor | None
    negative_prompt_embeds: torch.Tensor | None
    negative_pooled_prompt_embeds: torch.Tensor | None
    guidance_scale: float
    do_cfg: bool
    seed: int
    extra: dict[str, Any] = field(default_factory=dict)


def resolve_dtype(value: Any) -> torch.dtype:
    if isinstance(value, torch.dtype):
        return value
    table = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16,
             "float16": torch.float16, "fp32": torch.float32, "float32": torch.float32}
    key = str(value).replace("torch.", "")
    if key not in table:
        raise ValueError(f"unknown dtype {value!r}")
    return table[key]


@contextlib.contextmanager
def seeded_construction(seed: int, device: Any = None):
    """Inside the block the default random generators (CPU, and ``device`` when it is a GPU) are
    seeded with ``seed``; afterwards they are where they were.  Building a network inside it makes
    every weight a function of ``seed`` alone: the trainer's copy, a rollout worker's copy and
    every rank's copy come out identical, whatever was drawn before."""
    devices = []
    if device is not None:
        dev = torch.device(device)
        if dev.type == "cuda":
            devices = [dev.index if dev.index is not None else torch.cuda.current_device()]
    with torch.random.fork_rng(devices=devices):
        torch.manual_seed(int(seed))
        yield


def seeded_init(module: nn.Module, seed: int) -> None:
    """Re-draw every parameter of ``module`` from its own init law under a fixed seed.

    Construction already initialised the weights; this only makes the draw a
    function of ``seed`` so every rank (and every run) builds identical weights.
    """
    gens: dict = {}
    with torch.no_grad():
        for _, p in sorted(module.named_parameters()):
            if p.dim() >= 2:
                # draw on the parameter's own device: a 14B-parameter model is built directly in
                # HBM, never as an fp32 host copy
                gen = gens.get(p.device)
                if gen is None:
                    gen = gens[p.device] = torch.Generator(device=p.device).manual_seed(seed)
                std = float(p.float().std().item()) or 1.0 / math.sqrt(p.shape[-1])
                p.copy_(torch.randn(p.shape, generator=gen, device=p.device) * std)


class NativeFlowPolicy(DiffusionPolicy):
    """Base of the native diffusion families.

    Subclasses set ``family``, ``latent_rank`` (4 for images, 5 for video) and
    implement ``_build_modules(arch, spec)`` returning
    ``(transformer, decoder, text_encoder)`` plus ``_call_transformer``.
    """

    family = "flow"
    latent_rank = 4
    default_shift = 3.0
    context_length = 154

    def __init__(self, transformer: nn.Module, decoder: nn.Module | None, text_encoder: Any,
                 arch: dict[str, Any], device: Any, dtype: torch.dtype, shift: float | None = None):
        super().__init__()
        self.transformer = transformer
        object.__setattr__(self, "_frozen", SimpleNamespace(decoder=decoder, text=text_encoder))
        self.arch = dict(arch)
        self._device = torch.device(device)
        self._dtype = dtype
        self._scheduler = FlowMatchEulerScheduler(shift=shift if shift is not None
                                                  else self.default_shift)
        self._uses_lora = False

    # -- construction ---------------------------------------------------------------
    @classmethod
    def from_spec(cls, spec: Any) -> "NativeFlowPolicy":
        native = dict(spec.native_backend_config or {})
        arch = dict(native.get("arch") or {})
        if not arch:
            raise ValueError(f"{cls.__name__}.from_spec requires native_backend_config['arch']")
        dtype = resolve_dtype(spec.dtype)
        device = torch.device(spec.device)
        seed = int(native.get("init_seed", 0))
        # large networks are constructed where they will live (fp32 there, cast afterwards)
        # (seeded_init scales its draws by the spread of the weights it replaces, so the
        # construction itself has to be seeded as well; the decoder is only ever constructed)
        with seeded_construction(seed, device):
            with torch.device(device if device.type == "cuda" else "cpu"):
                transformer, decoder, text = cls._build_modules(arch, native)
            if native.get("random_init", True):
                seeded_init(transformer, seed)
        if not native.get("random_init", True):
            cls._load_native_checkpoint(transformer, spec.model_name_or_path)
        if native.get("text_encoder_path"):
            text = cls._build_prompt_encoder(str(native["text_encoder_path"]), arch, device)
        transformer.to(device=device, dtype=dtype)
        if decoder is not None:
            decoder.to(device=device, dtype=dtype if device.type == "cuda" else torch.float32)
            decoder.requires_grad_(False).eval()
        policy = cls(transformer, decoder, text, arch, device, dtype, native.get("shift"))
        steps = (spec.scheduler_config or {}).get("num_steps")
        if steps is not None:
            policy.set_num_steps(int(steps))
        return policy

    @staticmethod
    def _load_native_checkpoint(transformer: nn.Module, path: str) -> None:
        import os

        file = os.path.join(path, "transformer.safetensors")
        if not os.path.exists(file):
            raise FileNotFoundError(
                f"{file} not found: checkpoint-backed loading expects a directory in the native "
                "key layout; set model.random_init=true to build seeded random weights"
            )
        from safetensors.torch import load_file

        transformer.load_state_dict(load_file(file), strict=True)

    @classmethod
    def _build_modules(cls, arch: dict[str, Any], native: dict[str, Any]):
        raise NotImplementedError

    @classmethod
    def _build_prompt_encoder(cls, path: str, arch: dict[str, Any], device: torch.device):
        """The real text side from a local pipeline directory (``model.text_encoder.path``),
        replacing the seeded stand-in ``_build_modules`` returned."""
        raise NotImplementedError(f"{cls.__name__} has no checkpoint-backed prompt encoder")

    def _call_transformer(self, latents, timesteps, embeds, pooled, state):
        raise NotImplementedError

    # -- adapters / training mode ----------------------------------------------------
    def apply_lora(self, spec: Any) -> None:
        cfg = dict(spec.lora_config or {})
        apply_lora(self.transformer, int(cfg["rank"]), float(cfg["alpha"]),
                   list(cfg["target_modules"]), cfg.get("init", "gaussian"))
        self._uses_lora = True
        if spec.lora_path:
            self.load_lora_weights(spec.lora_path)

    def load_lora_weights(self, path: str) -> None:
        from visionrl_b200.models.nn.layers import load_lora_adapter

        load_lora_adapter(self.transformer, path)

    def enable_full_finetune(self) -> None:
        self.transformer.requires_grad_(True)
        self._uses_lora = False

    def torch_compile_transformer(self, mode: str) -> None:
        """Kept for configuration compatibility.  The launch-bound inner loops here are
        captured in CUDA graphs by the engine; no tracing compiler is involved."""
        self._graph_mode = mode

    def set_num_steps(self, n: int) -> None:
        self._scheduler.set_timesteps(int(n), device=self._device)

    @property
    def trainable_modules(self) -> dict[str, Any]:
        return {"transformer": self.transformer}

    @property
    def scheduler(self) -> Any:
        return self._scheduler

    @property
    def backend_handle(self) -> Any:
        return self._frozen

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def uses_lora(self) -> bool:
        return self._uses_lora

    # -- conditioning -----------------------------------------------------------------
    def encode_prompt(self, prompt, negative_prompt=None, **kwargs: Any) -> dict[str, Any]:
        length = int(kwargs.get("max_sequence_length", self.context_length))
        length = self._context_tokens(length)
        guidance = float(kwargs.get("guidance_scale", 4.5))
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        text = self._frozen.text
        emb, pooled = text(prompts, length, self._device, self._dtype)
        out = {"prompt_embeds": emb, "pooled_prompt_embeds": pooled,
               "negative_prompt_embeds": None, "negative_pooled_prompt_embeds": None}
        if guidance > 1.0:
            neg = negative_prompt if negative_prompt is not None else ""
            negs = [neg] * len(prompts) if isinstance(neg, str) else list(neg)
            out["negative_prompt_embeds"], out["negative_pooled_prompt_embeds"] = text(
                negs, length, self._device, self._dtype)
        if pooled is None:
            out.pop("pooled_prompt_embeds")
            out.pop("negative_pooled_prompt_embeds")
        return out

    def _context_tokens(self, max_sequence_length: int) -> int:
        return max_sequence_length

    # -- sampling ---------------------------------------------------------------------
    def latent_shape(self, request: VideoGenerationRequest) -> tuple:
        scale = int(self.arch.get("vae_scale", 8))
        ch = int(self.arch["in_channels"])
        if self.latent_rank == 4:
            return (ch, request.height // scale, request.width // scale)
        ts = int(self.arch.get("vae_temporal_scale", 4))
        return (ch, (request.frame_count - 1) // ts + 1, request.height // scale,
                request.width // scale)

    def prepare_sampling(self, request: VideoGenerationRequest, encoded: dict[str, Any],
                         **kwargs: Any) -> FlowSamplingState:
        self._scheduler.set_timesteps(request.num_steps, device=self._device)
        seed = request.seed if request.seed is not None else random.randint(0, sys.maxsize >> 1)
        gen = torch.Generator(device=self._device).manual_seed(int(seed))
        batch = encoded["prompt_embeds"].shape[0]
        latents = torch.randn((batch, *self.latent_shape(request)), generator=gen,
                              device=self._device, dtype=torch.float32)
        return FlowSamplingState(
            latents=latents, timesteps=self._scheduler.timesteps, scheduler=self._scheduler,
            prompt_embeds=encoded["prompt_embeds"],
            pooled_prompt_embeds=encoded.get("pooled_prompt_embeds"),
            negative_prompt_embeds=encoded.get("negative_prompt_embeds"),
            negative_pooled_prompt_embeds=encoded.get("negative_pooled_prompt_embeds"),
            guidance_scale=float(request.guidance_scale),
            do_cfg=request.guidance_scale > 1.0, seed=int(seed), extra=dict(kwargs),
        )

    # how the guidance combine reads: 0 = uncond + g (cond - uncond), 1 = cond + g (cond - uncond)
    cfg_form = 0

    def forward_step_raw(self, state: FlowSamplingState, step_idx: int):
        """The transformer output of one step BEFORE the guidance combine: ``(pred, do_cfg)`` with
        ``pred`` = ``[uncond ; cond]`` stacked along the batch when guidance is on, in the
        transformer's own dtype.  The rollout loop hands this to the fused SDE-step kernel, which
        does the combine, the step, the log-density and the trajectory write in one pass."""
        t = state.timesteps[step_idx]
        b = state.latents.shape[0]
        t_batch = t.expand(b) if t.ndim == 0 else t
        if not state.do_cfg:
            return self._call_transformer(state.latents, t_batch, state.prompt_embeds,
                                          state.pooled_prompt_embeds, state), False
        lat = torch.cat([state.latents, state.latents], dim=0)
        emb = torch.cat([state.negative_prompt_embeds, state.prompt_embeds], dim=0)
        pooled = None
        if state.pooled_prompt_embeds is not None:
            pooled = torch.cat([state.negative_pooled_prompt_embeds, state.pooled_prompt_embeds], dim=0)
        return self._call_transformer(lat, torch.cat([t_batch, t_batch]), emb, pooled, state), True

    def forward_step(self, state: FlowSamplingState, step_idx: int) -> dict[str, Any]:
        out, do_cfg = self.forward_step_raw(state, step_idx)
        if do_cfg:
            uncond, cond = out.float().chunk(2, dim=0)
            noise_pred = self._combine_cfg(cond, uncond, state.guidance_scale)
        else:
            cond = out.float()
            uncond = torch.zeros_like(cond)
            noise_pred = cond
        return {"noise_pred": noise_pred, "noise_pred_cond": cond, "noise_pred_uncond": uncond}

    @staticmethod
    def _combine_cfg(cond, uncond, scale: float):
        return uncond + scale * (cond - uncond)

    def decode_latents(self, latents: torch.Tensor) -> torch.Tensor:
        decoder = self._frozen.decoder
        if decoder is None:
            return latents
        with torch.no_grad():
            image = decoder(latents)
        return (image.float() / 2 + 0.5).clamp(0, 1)

    # -- collector boundary --------------------------------------------------------------
    def export_batch_context(self, state: FlowSamplingState) -> dict[str, Any]:
        return {"guidance_scale": state.guidance_scale, "cfg": state.do_cfg,
                "model_family": self.family}

    def export_training_extras(self, state: FlowSamplingState) -> dict[str, Any]:
        out = {"prompt_embeds": state.prompt_embeds,
               "negative_prompt_embeds": state.negative_prompt_embeds}
        if state.pooled_prompt_embeds is not None:
            out["pooled_prompt_embeds"] = state.pooled_prompt_embeds
            out["negative_pooled_prompt_embeds"] = state.negative_pooled_prompt_embeds
        return out

    def restore_eval_state(self, batch_extras, batch_context, latents, step_idx) -> FlowSamplingState:
        ts = batch_extras["timesteps"]
        t = ts[:, step_idx] if ts.ndim > 1 else ts
        guidance = float(batch_context["guidance_scale"])
        return FlowSamplingState(
            latents=latents, timesteps=t.unsqueeze(0) if t.ndim == 1 else t, scheduler=None,
            prompt_embeds=batch_extras["prompt_embeds"],
            pooled_prompt_embeds=batch_extras.get("pooled_prompt_embeds"),
            negative_prompt_embeds=batch_extras.get("negative_prompt_embeds"),
            negative_pooled_prompt_embeds=batch_extras.get("negative_pooled_prompt_embeds"),
            guidance_scale=guidance, do_cfg=bool(batch_context["cfg"]) and guidance > 1.0, seed=0,
        )
