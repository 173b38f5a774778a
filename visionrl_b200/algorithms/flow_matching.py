"""Flow-matching SDE / CPS step with its Gaussian log-probability.

One function serves the rollout (draws ``prev_sample``) and the training replay
(``prev_sample`` given, gradients flow to ``model_output``).  All math is fp32.
With ``sigma`` the current and ``sigma'`` the next noise level, ``dt = sigma' -
sigma < 0``, ``v`` the model output and ``x`` the sample:

``sde``:  ``s = sqrt(sigma / (1 - sigma*)) * noise_level`` (``sigma* = sigma``,
          or ``sigmas[1]`` where ``sigma == 1``); for ``noise_level == 1`` the
          linear form ``s = sigma_min + (sigma_max - sigma_min) * sigma`` is used;
          ``mu = x (1 + s^2/(2 sigma) dt) + v (1 + s^2 (1-sigma)/(2 sigma)) dt``;
          ``x' = mu + s sqrt(-dt) eps``;
          ``logp = mean(-(x'-mu)^2 / (2 nu^2) - log nu - log sqrt(2 pi))``, ``nu = s sqrt(-dt)``.
``cps``:  ``s = sigma' sin(noise_level pi/2)``; ``x0 = x - sigma v``; ``n = x + (1-sigma) v``;
          ``mu = x0 (1-sigma') + n sqrt(sigma'^2 - s^2)``; ``x' = mu + s eps``;
          ``logp = mean(-(x'-mu)^2)``.

``sigma_max`` is ``sigmas[1]`` and ``sigma_min`` is ``sigmas[-1]`` (reference:
``vrl/algorithms/flow_matching.py:21-149``).  On CUDA tensors the element-wise
part runs in the fused sm_100a kernel of :mod:`visionrl_b200.ops.sde`.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any


@dataclass(slots=True)
class SDEStepResult:
    prev_sample: Any
    log_prob: Any
    prev_sample_mean: Any
    std_dev_t: Any
    dt: Any | None = None


def randn_tensor(shape, generator=None, device=None, dtype=None):
    """Gaussian noise honouring a generator that may live on another device."""
    import torch

    device = torch.device(device) if device is not None else torch.device("cpu")
    if isinstance(generator, (list, tuple)):
        parts = [randn_tensor((1, *shape[1:]), g, device, dtype) for g in generator]
        return torch.cat(parts, dim=0)
    if generator is not None and generator.device.type != device.type:
        noise = torch.randn(shape, generator=generator, device=generator.device, dtype=dtype)
        return noise.to(device)
    return torch.randn(shape, generator=generator, device=device, dtype=dtype)


def step_coefficients(sigmas, step_index, noise_level: float, sde_type: str):
    """Per-sample scalars ``(a, b, std_dev_t, noise_scale, sqrt(-dt), dt)`` with ``mu = a x + b v``.

    ``sigmas`` is the scheduler's 1-D schedule (trailing 0 included) and
    ``step_index`` a ``[B]`` long tensor.  Everything is computed in fp32 with the
    same operation order as the element-wise formulas in the module docstring.
    """
    import torch

    sigmas = sigmas.to(dtype=torch.float32)
    sigma = sigmas[step_index]
    sigma_next = sigmas[step_index + 1]
    sigma_max = sigmas[1]
    sigma_min = sigmas[-1]
    dt = sigma_next - sigma
    if sde_type == "cps":
        std = sigma_next * math.sin(noise_level * math.pi / 2)
        root = torch.sqrt(sigma_next**2 - std**2)
        a = (1 - sigma_next) + root
        b = -sigma * (1 - sigma_next) + (1 - sigma) * root
        scale = std
    elif sde_type == "sde":
        if noise_level != 1.0:
            denom = 1 - torch.where(sigma == 1, sigma_max, sigma)
            std = torch.sqrt(sigma / denom) * noise_level
        else:
            std = sigma_min + (sigma_max - sigma_min) * sigma
        a = 1 + std**2 / (2 * sigma) * dt
        b = (1 + std**2 * (1 - sigma) / (2 * sigma)) * dt
        scale = std * torch.sqrt(-dt)
    else:
        raise ValueError(f"unknown sde_type {sde_type!r}; expected 'sde' or 'cps'")
    return a, b, std, scale, torch.sqrt(-dt), dt


def _step_indices(scheduler: Any, timestep: Any, device):
    import torch

    if hasattr(scheduler, "indices_for_timesteps"):
        return scheduler.indices_for_timesteps(timestep).to(device)
    return torch.as_tensor(
        [int(scheduler.index_for_timestep(t)) for t in timestep], dtype=torch.long, device=device
    )


def sde_step_with_logprob(
    scheduler: Any,
    model_output: Any,
    timestep: Any,
    sample: Any,
    prev_sample: Any | None = None,
    generator: Any | None = None,
    deterministic: bool = False,
    return_dt: bool = False,
    noise_level: float = 1.0,
    sde_type: str = "sde",
) -> SDEStepResult:
    import torch

    from visionrl_b200.ops import sde as sde_ops

    if prev_sample is not None and generator is not None:
        raise ValueError("Cannot pass both generator and prev_sample.")
    model_output = model_output.float()
    sample = sample.float()
    device = sample.device
    sigmas = scheduler.sigmas.to(device)
    scheduler.sigmas = sigmas
    index = _step_indices(scheduler, timestep, device)
    a, b, std, scale, sqrt_neg_dt, dt = step_coefficients(sigmas, index, noise_level, sde_type)
    view = (-1,) + (1,) * (sample.ndim - 1)

    noise = None
    if prev_sample is None:
        noise = randn_tensor(model_output.shape, generator, device, torch.float32)
    else:
        prev_sample = prev_sample.float()
    out_prev, log_prob, mean = sde_ops.sde_step(
        model_output, sample, a, b, scale, dt,
        prev_sample=prev_sample, noise=noise, deterministic=deterministic,
        gaussian=(sde_type == "sde"),
    )
    return SDEStepResult(
        prev_sample=out_prev,
        log_prob=log_prob,
        prev_sample_mean=mean,
        std_dev_t=std.view(view),
        dt=sqrt_neg_dt.view(view) if return_dt else None,
    )


def compute_kl_divergence(prev_sample_mean, prev_sample_mean_ref, std_dev_t, dt=None):
    """``mean((mu - mu_ref)^2) / (2 s^2)``, or ``/(2 (s dt)^2)`` when ``dt`` is passed."""
    denom = 2 * std_dev_t**2 if dt is None else 2 * (std_dev_t * dt) ** 2
    dims = tuple(range(1, prev_sample_mean.ndim))
    return ((prev_sample_mean - prev_sample_mean_ref) ** 2).mean(dim=dims) / denom.squeeze()


__all__ = [
    "SDEStepResult",
    "compute_kl_divergence",
    "randn_tensor",
    "sde_step_with_logprob",
    "step_coefficients",
]
