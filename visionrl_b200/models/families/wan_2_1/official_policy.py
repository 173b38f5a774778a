"""Wan variant with two timestep experts, sequential CFG and the multistep flow solvers.

A high-noise and a low-noise transformer are switched at a boundary timestep
(``boundary * num_train_timesteps``); conditional and unconditional branches run as two
forwards; encoded prompts are cached by a SHA-256 key.  ``request.sample_solver`` picks the
deterministic sampler of :meth:`sample`: ``"unipc"`` (UniPC) or anything else, by default
``"dpmpp"`` (DPM-Solver++ 2M), both from :mod:`visionrl_b200.models.nn.flow_solvers` on the
shifted uniform grid of ``request.shift``.  As in the reference
(``vrl/models/families/wan_2_1/official_policy.py:65-602``, solver choice at ``:453-478``) this
variant is rollout-only: it has no adapter path and ``restore_eval_state`` raises.
"""

from __future__ import annotations

import copy
import hashlib
from typing import Any

import torch

from visionrl_b200.models.families.wan_2_1.diffusers_policy import WanSamplingState, WanT2VDiffusersPolicy


class WanT2VOfficialPolicy(WanT2VDiffusersPolicy):
    family = "wan_2_1"

    def __init__(self, *args: Any, boundary: float = 0.875, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self.boundary = boundary
        object.__setattr__(self, "_low_noise", None)
        self._prompt_cache: dict[str, dict[str, Any]] = {}

    @classmethod
    def from_spec(cls, spec: Any) -> "WanT2VOfficialPolicy":
        """``model.backend: official`` builds this variant: ``model.arch.boundary`` sets the switch
        point and, unless ``model.arch.two_experts`` is false, the low-noise expert is attached
        (with random init: a second network drawn from ``init_seed + 1``)."""
        policy = super().from_spec(spec)
        native = dict(spec.native_backend_config or {})
        arch = dict(native.get("arch") or {})
        policy.boundary = float(arch.get("boundary", policy.boundary))
        if bool(arch.get("two_experts", True)):
            expert = None
            if native.get("random_init", True):
                from visionrl_b200.models.families.flow_policy import seeded_construction, seeded_init

                seed = int(native.get("init_seed", 0)) + 1
                with seeded_construction(seed, policy.device):
                    expert = copy.deepcopy(policy.transformer)
                    seeded_init(expert, seed)
            policy.attach_low_noise_expert(expert)
        return policy

    def attach_low_noise_expert(self, module: torch.nn.Module | None = None) -> None:
        expert = module if module is not None else copy.deepcopy(self.transformer)
        object.__setattr__(self, "_low_noise", expert.requires_grad_(False).eval())

    def _expert(self, t: torch.Tensor):
        low = self._low_noise
        if low is None:
            return self.transformer
        threshold = self.boundary * self._scheduler.num_train_timesteps
        return self.transformer if float(t.flatten()[0]) >= threshold else low

    def encode_prompt(self, prompt, negative_prompt=None, **kwargs: Any) -> dict[str, Any]:
        key = hashlib.sha256(repr((prompt, negative_prompt, kwargs.get("max_sequence_length"),
                                   kwargs.get("guidance_scale"))).encode()).hexdigest()
        if key not in self._prompt_cache:
            self._prompt_cache[key] = super().encode_prompt(prompt, negative_prompt, **kwargs)
        return dict(self._prompt_cache[key])

    def forward_step(self, state, step_idx: int) -> dict[str, Any]:
        t = state.timesteps[step_idx]
        b = state.latents.shape[0]
        t_batch = t.expand(b) if t.ndim == 0 else t
        net = self._expert(t_batch)
        cond = net(state.latents, t_batch, state.prompt_embeds).float()
        if state.do_cfg:
            uncond = net(state.latents, t_batch, state.negative_prompt_embeds).float()
            noise_pred = uncond + state.guidance_scale * (cond - uncond)
        else:
            uncond, noise_pred = torch.zeros_like(cond), cond
        return {"noise_pred": noise_pred, "noise_pred_cond": cond, "noise_pred_uncond": uncond}

    def build_solver(self, request: Any):
        """The ODE solver ``request.sample_solver`` names, configured for ``request.num_steps``."""
        from visionrl_b200.models.nn import flow_solvers as fs

        train_steps = int(self._scheduler.num_train_timesteps)
        shift = float(getattr(request, "shift", 1.0) or 1.0)
        if str(getattr(request, "sample_solver", "dpmpp")) == "unipc":
            solver = fs.FlowUniPCMultistepScheduler(num_train_timesteps=train_steps, shift=1.0)
            solver.set_timesteps(int(request.num_steps), device=self._device, shift=shift)
        else:
            solver = fs.FlowDPMSolverMultistepScheduler(num_train_timesteps=train_steps, shift=1.0)
            fs.retrieve_timesteps(solver, device=self._device,
                                  sigmas=fs.get_sampling_sigmas(int(request.num_steps), shift))
        return solver

    @torch.no_grad()
    def sample(self, request: Any, encoded: dict[str, Any] | None = None, decode: bool = True):
        """Deterministic generation with the requested multistep solver (no log-probabilities:
        this is the preview / evaluation sampler, not the SDE rollout)."""
        if encoded is None:
            encoded = self.encode_prompt(request.prompt, request.negative_prompt or None,
                                         guidance_scale=request.guidance_scale, request=request)
        state = self.prepare_sampling(request, encoded)
        solver = self.build_solver(request)
        state.scheduler, state.timesteps = solver, solver.timesteps
        for i, t in enumerate(solver.timesteps):
            pred = self.forward_step(state, i)["noise_pred"]
            state.latents = solver.step(pred, t, state.latents)
        return self.decode_latents(state.latents) if decode else state.latents

    def apply_lora(self, spec: Any) -> None:
        raise NotImplementedError("the two-expert Wan variant has no adapter path")

    def restore_eval_state(self, batch_extras, batch_context, latents, step_idx):
        raise NotImplementedError("the two-expert Wan variant is rollout-only (no replay path)")


WanT2VOfficialSamplingState = WanSamplingState

__all__ = ["WanT2VOfficialPolicy", "WanT2VOfficialSamplingState"]
