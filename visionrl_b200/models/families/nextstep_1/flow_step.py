"""Per-token flow-matching sampler with a Gaussian log-probability (math of kernel family M10).

One continuous token is produced by integrating the head's velocity field from ``x_0 ~ N(0, I)``
on the grid ``t_k = k/K``: ``K-1`` deterministic Euler steps ``x += dt * v``, then a final step
``mu = x + dt * v`` followed by ``token = mu + std * eps`` with ``std = noise_level * sqrt(dt)``.
With CFG the velocity is ``(1 + s) v(x, cond) - s v(x, uncond)``.  The log-probability is the
isotropic Gaussian density summed over the ``D`` token channels,
``-|token - mu|^2 / (2 std^2) - D log std - (D/2) log 2 pi``.  Replaying with the saved
``x_0`` reproduces the rollout value exactly (reference:
``vrl/models/families/nextstep_1/flow_step.py:30-275``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass(slots=True)
class FlowStepResult:
    token: torch.Tensor
    log_prob: torch.Tensor
    mean: torch.Tensor
    std: torch.Tensor
    initial_noise: torch.Tensor


def _velocity_fn(image_head: Any, velocity_fn: Callable | None) -> Callable:
    if velocity_fn is not None:
        return velocity_fn
    net = getattr(image_head, "net", None)
    return net if net is not None else image_head


def _integrate(velocity, x, cond, uncond, cfg_scale: float, steps: int):
    """Deterministic prefix + final mean.  Returns ``mu``."""
    b = x.shape[0]
    dt = 1.0 / steps
    grid = torch.linspace(0.0, 1.0, steps + 1, device=x.device, dtype=x.dtype)
    guided = uncond is not None and abs(cfg_scale - 1.0) > 1e-6
    for k in range(steps):
        tk = grid[k].expand(b)
        v = velocity(x, tk, cond)
        if guided:
            v = (1.0 + cfg_scale) * v - cfg_scale * velocity(x, tk, uncond)
        x = x + dt * v
    return x


def gaussian_token_log_prob(token, mean, std: float):
    d = token.shape[-1]
    sq = ((token.detach() - mean) ** 2).sum(dim=-1)
    return (-sq / (2.0 * std**2) - float(d) * math.log(max(std, 1e-12))
            - 0.5 * float(d) * math.log(2.0 * math.pi))


def flow_sample_with_logprob(image_head: Any, cond: torch.Tensor, *, num_flow_steps: int = 20,
                             noise_level: float = 1.0, cfg_uncond: torch.Tensor | None = None,
                             cfg_scale: float = 1.0, generator: torch.Generator | None = None,
                             initial_noise: torch.Tensor | None = None,
                             velocity_fn: Callable | None = None,
                             final_noise: torch.Tensor | None = None) -> FlowStepResult:
    token_dim = getattr(image_head, "input_dim", None)
    if token_dim is None:
        raise RuntimeError("flow_sample_with_logprob: image_head has no ``input_dim`` attribute")
    b, d = cond.shape[0], int(token_dim)
    if initial_noise is None:
        x0 = torch.randn(b, d, device=cond.device, dtype=cond.dtype, generator=generator)
    else:
        if tuple(initial_noise.shape) != (b, d):
            raise ValueError(f"initial_noise must have shape {(b, d)}, got {tuple(initial_noise.shape)}")
        x0 = initial_noise.to(device=cond.device, dtype=cond.dtype)
    mean = _integrate(_velocity_fn(image_head, velocity_fn), x0, cond, cfg_uncond, cfg_scale,
                      num_flow_steps)
    std = noise_level * math.sqrt(1.0 / num_flow_steps)
    eps = final_noise if final_noise is not None else torch.randn(
        mean.shape, device=mean.device, dtype=mean.dtype, generator=generator)
    token = mean + std * eps
    return FlowStepResult(token=token, log_prob=gaussian_token_log_prob(token, mean, std), mean=mean,
                          std=torch.full((b,), std, device=cond.device, dtype=cond.dtype),
                          initial_noise=x0)


def flow_logprob_at(image_head: Any, cond: torch.Tensor, target_token: torch.Tensor,
                    saved_noise: torch.Tensor | None = None, *, num_flow_steps: int = 20,
                    noise_level: float = 1.0, cfg_uncond: torch.Tensor | None = None,
                    cfg_scale: float = 1.0, velocity_fn: Callable | None = None) -> torch.Tensor:
    """Log-probability of ``target_token`` under the current head; gradients reach the head."""
    b, d = target_token.shape
    if saved_noise is not None:
        x0 = saved_noise.to(device=target_token.device, dtype=target_token.dtype)
    else:
        x0 = torch.randn(b, d, device=target_token.device, dtype=target_token.dtype)
    mean = _integrate(_velocity_fn(image_head, velocity_fn), x0, cond, cfg_uncond, cfg_scale,
                      num_flow_steps)
    return gaussian_token_log_prob(target_token, mean, noise_level * math.sqrt(1.0 / num_flow_steps))


__all__ = ["FlowStepResult", "flow_logprob_at", "flow_sample_with_logprob",
           "gaussian_token_log_prob"]
