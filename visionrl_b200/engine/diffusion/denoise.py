"""One diffusion micro-batch: prepare → T denoise steps with log-probs → decode.

The latent trajectory is kept in a single ``[b, T+1, ...]`` fp32 buffer on the
device; ``observations`` (``x_t`` before each step) and ``actions`` (``x_{t-1}``
after it) are the two shifted views of that buffer, so nothing is cloned or
stacked inside the loop and nothing leaves the GPU.  Per step the policy runs
one (CFG-batched) transformer forward and the SDE math runs in
:func:`visionrl_b200.algorithms.flow_matching.sde_step_with_logprob`
(reference loop: ``vrl/engine/diffusion/denoise.py:77-165``).  The recorded
``kl`` is ``|log_prob|`` when ``return_kl`` is set and 0 otherwise — a shaping
signal, not a divergence.
"""

from __future__ import annotations

import random
from dataclasses import dataclass
from typing import Any

import torch

from visionrl_b200.algorithms.flow_matching import sde_step_with_logprob, step_coefficients
from visionrl_b200.engine.core.protocols import PipelineChunkResult
from visionrl_b200.engine.core.types import (
    GenerationMetrics, GenerationRequest, GenerationSampleSpec, OutputBatch,
    RolloutDenoisingEnv, RolloutDitTrajectory, RolloutTrajectoryData,
)


@dataclass(frozen=True, slots=True)
class DiffusionDenoiseConfig:
    sample_start: int
    seed: int | None
    same_latent: bool
    sde_window: tuple[int, int] | None
    return_kl: bool
    noise_level: float = 1.0
    sde_type: str = "sde"


@dataclass(slots=True)
class DiffusionChunkResult(PipelineChunkResult):
    observations: Any
    actions: Any
    log_probs: Any
    timesteps: Any
    kl: Any
    video: Any
    training_extras: dict[str, Any]
    context: dict[str, Any]


def select_sde_window(sde_window_size: int, sde_window_range, rng: random.Random | None = None):
    """Random window of stochastic steps; ``None`` means every step is stochastic."""
    if sde_window_size <= 0:
        return None
    lo, hi = int(sde_window_range[0]), int(sde_window_range[1])
    start = (rng or random).randint(lo, max(lo, hi - sde_window_size))
    return (start, start + sde_window_size)


def repeat_tensor_batch(value: Any, count: int) -> Any:
    if count < 1:
        raise ValueError("count must be >= 1")
    if not isinstance(value, torch.Tensor) or count == 1:
        return value
    return value.repeat(count, *([1] * (value.ndim - 1)))


def _chunk_generator(device, sample_start: int, seed: int | None, same_latent: bool):
    if seed is None:
        if same_latent:
            raise ValueError("same_latent=True requires an explicit sampling.seed")
        return None
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + sample_start)
    return gen


# The fused rollout step (guidance combine + SDE step + log-density + trajectory write in one
# kernel, noise from Philox keyed by the chunk's seed) is used whenever the policy can hand over its
# raw transformer output; set to False to force the generic path (separate combine, torch.randn).
FUSED_ROLLOUT_STEP = True


def _fused_step_available(policy: Any, path: torch.Tensor) -> bool:
    from visionrl_b200.ops import _ext

    n = path[0, 0].numel()
    return (FUSED_ROLLOUT_STEP and path.is_cuda and n % 4 == 0 and path.shape[0] <= 65535
            and callable(getattr(policy, "forward_step_raw", None))
            and type(policy).forward_step is _base_forward_step(policy)
            and _ext.kernels_enabled() and _ext.has("sde_rollout_step"))


def _base_forward_step(policy: Any):
    """``forward_step`` of the class that defines ``forward_step_raw``: a subclass that overrides
    ``forward_step`` (other guidance algebra, preconditioning) must take the generic path."""
    for klass in type(policy).__mro__:
        if "forward_step_raw" in klass.__dict__:
            return klass.__dict__.get("forward_step")
    return None


def _philox_seed(config: "DiffusionDenoiseConfig") -> int:
    if config.seed is not None:
        return (int(config.seed) + int(config.sample_start)) & 0x7FFFFFFFFFFFFFFF
    # unseeded requests follow the process-wide generator, like torch.randn would
    return int(torch.randint(0, 2**62, (1,), dtype=torch.int64).item())


def run_diffusion_denoise_chunk(*, policy: Any, request: Any, encoded: dict[str, Any],
                                config: DiffusionDenoiseConfig,
                                prepare_kwargs: dict[str, Any] | None = None) -> DiffusionChunkResult:
    state = policy.prepare_sampling(request, encoded, **(prepare_kwargs or {}))
    latents0 = state.latents
    b, device = latents0.shape[0], latents0.device
    steps = len(state.timesteps)
    generator = _chunk_generator(device, config.sample_start, config.seed, config.same_latent)

    path = torch.empty((b, steps + 1, *latents0.shape[1:]), dtype=torch.float32, device=device)
    path[:, 0] = latents0
    log_probs = torch.empty((b, steps), dtype=torch.float32, device=device)
    fused = _fused_step_available(policy, path)
    if fused:
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        seed = _philox_seed(config)
        sigmas = state.scheduler.sigmas.to(device)
        state.scheduler.sigmas = sigmas

    with torch.no_grad():
        for i in range(steps):
            state.latents = path[:, i]
            stochastic = config.sde_window is None or config.sde_window[0] <= i < config.sde_window[1]
            if fused:
                pred, has_cfg = policy.forward_step_raw(state, i)
                index = torch.full((b,), i, dtype=torch.long, device=device)
                ca, cb, _std, scale, _sq, dt = step_coefficients(sigmas, index, config.noise_level,
                                                                 config.sde_type)
                ext.sde_rollout_step(pred.contiguous(), bool(has_cfg), float(state.guidance_scale),
                                     int(getattr(policy, "cfg_form", 0)), path, i, ca.contiguous(),
                                     cb.contiguous(), scale.contiguous(), dt.contiguous(), None, seed,
                                     4 * i, log_probs, not stochastic, config.sde_type == "sde")
                continue
            noise_pred = policy.forward_step(state, i)["noise_pred"]
            res = sde_step_with_logprob(
                state.scheduler, noise_pred, state.timesteps[i].reshape(1).expand(b), path[:, i],
                generator=generator if stochastic else None, deterministic=not stochastic,
                return_dt=config.return_kl, noise_level=config.noise_level,
                sde_type=config.sde_type,
            )
            path[:, i + 1] = res.prev_sample
            log_probs[:, i] = res.log_prob
        state.latents = path[:, steps]
        video = policy.decode_latents(state.latents)

    timesteps = state.timesteps.to(device).reshape(1, steps).expand(b, steps).contiguous()
    kl = log_probs.abs() if config.return_kl else torch.zeros_like(log_probs)
    return DiffusionChunkResult(
        observations=path[:, :-1], actions=path[:, 1:], log_probs=log_probs, timesteps=timesteps,
        kl=kl, video=video, training_extras=policy.export_training_extras(state),
        context=policy.export_batch_context(state),
    )


def _cat_extras(parts: list[dict[str, Any]]) -> dict[str, Any]:
    out: dict[str, Any] = {}
    for key in (parts[0] if parts else {}):
        vals = [p[key] for p in parts]
        if any(v is None for v in vals):
            out[key] = None
        elif all(isinstance(v, torch.Tensor) for v in vals):
            out[key] = torch.cat(vals, dim=0)
        else:
            out[key] = vals[0]
    return out


def peak_memory_mb() -> float | None:
    if not torch.cuda.is_available():
        return None
    try:
        return torch.cuda.max_memory_allocated() / (1024 * 1024)
    except Exception:  # noqa: BLE001
        return None


def build_diffusion_output_batch(*, request: GenerationRequest,
                                 sample_specs: list[GenerationSampleSpec], prompts: list[str],
                                 chunks: list[DiffusionChunkResult], num_steps: int) -> OutputBatch:
    if not chunks:
        raise ValueError("chunks must be non-empty")
    context = chunks[0].context
    if not context:
        raise ValueError("DiffusionChunkResult.context must be non-empty")
    cat = lambda name: torch.cat([getattr(c, name) for c in chunks], dim=0)  # noqa: E731
    observations, actions = cat("observations"), cat("actions")
    video = cat("video")
    env = RolloutDenoisingEnv(extra={
        "actions": actions, "kl": cat("kl"),
        "training_extras": _cat_extras([c.training_extras for c in chunks]),
        "context": context, "videos": video,
    })
    data = RolloutTrajectoryData(
        rollout_log_probs=cat("log_probs"), denoising_env=env,
        dit_trajectory=RolloutDitTrajectory(latents=observations, timesteps=cat("timesteps")),
    )
    peak = peak_memory_mb()
    return OutputBatch(
        request_id=request.request_id, family=request.family, task=request.task, prompts=prompts,
        sample_specs=sample_specs, output=video, rollout_trajectory_data=data,
        metrics=GenerationMetrics(num_prompts=len(prompts), num_samples=len(sample_specs),
                                  num_steps=num_steps, micro_batches=len(chunks),
                                  peak_memory_mb=peak),
        peak_memory_mb=peak or 0.0,
    )


__all__ = [
    "DiffusionChunkResult", "DiffusionDenoiseConfig", "build_diffusion_output_batch",
    "peak_memory_mb", "repeat_tensor_batch", "run_diffusion_denoise_chunk", "select_sde_window",
]
