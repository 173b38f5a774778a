"""Guided categorical sampling of image tokens (kernel K10 and its oracle).

``guided = uncond + w (cond - uncond)``; the token is drawn from ``softmax(guided / T)`` by
inverse-CDF search with a given uniform variate per row (so the draw is a pure function of the
logits and ``u``), and the recorded log-probability is ``log_softmax(cond / T)[token]`` — the
conditional, unguided distribution.
"""

from __future__ import annotations

import torch


def sample_cfg_tokens_reference(cond, uncond, u, cfg_weight: float, temperature: float):
    cond_f, uncond_f = cond.float(), uncond.float()
    guided = uncond_f + cfg_weight * (cond_f - uncond_f)
    probs = torch.softmax(guided / temperature, dim=-1)
    cdf = torch.cumsum(probs, dim=-1)
    target = (u.float().clamp(0.0, 1.0 - 1e-7) * cdf[:, -1]).unsqueeze(-1)
    tokens = (cdf <= target).sum(dim=-1).clamp(max=cond.shape[-1] - 1)
    log_probs = torch.log_softmax(cond_f / temperature, dim=-1).gather(-1, tokens[:, None])[:, 0]
    return tokens, log_probs


def sample_cfg_tokens(cond, uncond, u, cfg_weight: float, temperature: float):
    """``cond``/``uncond`` ``[R, V]`` logits, ``u[R]`` uniforms → ``(tokens[R], log_probs[R])``."""
    from visionrl_b200.ops import _ext

    if cond.is_cuda and _ext.kernels_enabled() and _ext.has("sample_tokens"):
        return _ext.load().sample_tokens(cond.contiguous(), uncond.contiguous(),
                                         u.contiguous().float(), float(cfg_weight),
                                         float(temperature))
    return sample_cfg_tokens_reference(cond, uncond, u, cfg_weight, temperature)
