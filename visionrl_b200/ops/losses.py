"""Policy-gradient and preference losses (kernels K6 / K14 and their oracles).

Every function returns graph-attached loss tensors plus detached metric tensors
that stay on the device; nothing here calls ``.item()``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from visionrl_b200.ops import _ext


def grpo_clipped_loss_reference(log_prob, old_log_prob, advantages, eps_clip: float):
    ratio = torch.exp(log_prob - old_log_prob)
    clipped = torch.clamp(ratio, 1.0 - eps_clip, 1.0 + eps_clip)
    loss = torch.mean(torch.maximum(-advantages * ratio, -advantages * clipped))
    with torch.no_grad():
        clip_fraction = (torch.abs(ratio - 1.0) > eps_clip).float().mean()
        approx_kl = 0.5 * torch.mean((log_prob - old_log_prob) ** 2)
    return loss, clip_fraction, approx_kl


def token_grpo_loss_reference(log_prob, old_log_prob, advantages, mask, ref_log_prob,
                              eps_clip: float, kl_estimator: str):
    if mask is None:
        mask = torch.ones_like(log_prob)
    mask = mask.to(dtype=log_prob.dtype, device=log_prob.device)
    adv = advantages.unsqueeze(-1).expand_as(log_prob) if advantages.dim() == 1 else advantages
    ratio = torch.exp(log_prob - old_log_prob)
    clipped = torch.clamp(ratio, 1.0 - eps_clip, 1.0 + eps_clip)
    per_token = torch.maximum(-adv * ratio, -adv * clipped)
    denom = mask.sum().clamp_min(1.0)
    policy_loss = (per_token * mask).sum() / denom
    if ref_log_prob is not None:
        delta = log_prob - ref_log_prob
        kl_tok = torch.exp(delta) * (delta - 1.0) + 1.0 if kl_estimator == "k3" else delta
        kl_loss = (kl_tok * mask).sum() / denom
    else:
        kl_loss = torch.zeros((), device=log_prob.device)
    with torch.no_grad():
        valid = (mask > 0).to(log_prob.dtype)
        n_valid = valid.sum().clamp_min(1.0)
        clip_fraction = ((torch.abs(ratio - 1.0) > eps_clip).to(log_prob.dtype) * valid).sum() / n_valid
        approx_kl = 0.5 * (((log_prob - old_log_prob) ** 2) * valid).sum() / n_valid
    return policy_loss, kl_loss, clip_fraction, approx_kl


class _FusedTokenLoss(torch.autograd.Function):
    """One pass over ``[B, L]``: surrogate, KL, metrics and d(loss)/d(log_prob)."""

    @staticmethod
    def forward(ctx, log_prob, old_log_prob, advantages, mask, ref_log_prob, eps_clip, k3):
        from visionrl_b200.ops import _ext

        out, g_pol, g_kl = _ext.load().token_loss_fwd(
            log_prob.contiguous(), old_log_prob.contiguous(), advantages.contiguous(),
            None if mask is None else mask.contiguous().float(),
            None if ref_log_prob is None else ref_log_prob.contiguous(), float(eps_clip), bool(k3),
        )
        ctx.save_for_backward(g_pol, g_kl)
        return out[0], out[1], out[2], out[3]

    @staticmethod
    def backward(ctx, g_policy, g_kl_loss, _gc, _ga):
        g_pol, g_kl = ctx.saved_tensors
        grad = g_pol * g_policy
        if g_kl_loss is not None:
            grad = grad + g_kl * g_kl_loss
        return grad, None, None, None, None, None, None


def grpo_clipped_loss(log_prob, old_log_prob, advantages, eps_clip: float):
    """``log_prob[B]`` → ``(policy_loss, clip_fraction, approx_kl)``."""
    if (log_prob.is_cuda and log_prob.dim() == 1 and log_prob.dtype == torch.float32
            and _ext.kernels_enabled()):
        b = log_prob.shape[0]
        pol, _kl, clip, akl = _FusedTokenLoss.apply(
            log_prob.view(b, 1), old_log_prob.view(b, 1).float(), advantages.float(), None, None,
            eps_clip, True,
        )
        return pol, clip.detach(), akl.detach()
    return grpo_clipped_loss_reference(log_prob, old_log_prob, advantages, eps_clip)


def token_grpo_loss(log_prob, old_log_prob, advantages, mask, ref_log_prob, eps_clip: float,
                    kl_estimator: str = "k3"):
    """``log_prob[B, L]`` → ``(policy_loss, kl_loss, clip_fraction, approx_kl)``."""
    if (log_prob.is_cuda and log_prob.dim() == 2 and advantages.dim() == 1
            and log_prob.dtype == torch.float32 and _ext.kernels_enabled()):
        pol, kl, clip, akl = _FusedTokenLoss.apply(
            log_prob, old_log_prob.float(), advantages.float(), mask, ref_log_prob, eps_clip,
            kl_estimator == "k3",
        )
        return pol, kl, clip.detach(), akl.detach()
    return token_grpo_loss_reference(
        log_prob, old_log_prob, advantages, mask, ref_log_prob, eps_clip, kl_estimator
    )


def per_sample_mse(pred, target):
    """``mean((pred - target)^2)`` over all non-batch dims, fp32 accumulation."""
    if (pred.is_cuda and not (pred.requires_grad or target.requires_grad)
            and _ext.kernels_enabled()):
        return _ext.load().per_sample_mse(pred.contiguous(), target.contiguous())
    return (pred.float() - target.float()).pow(2).mean(dim=tuple(range(1, pred.ndim)))


def dpo_loss_reference(model_pred, ref_pred, target, beta: float):
    dims = tuple(range(1, model_pred.ndim))
    model_losses = (model_pred - target).pow(2).mean(dim=dims)
    win, lose = model_losses.chunk(2)
    with torch.no_grad():
        ref_losses = (ref_pred - target).pow(2).mean(dim=dims)
        ref_w, ref_l = ref_losses.chunk(2)
    model_diff = win - lose
    ref_diff = ref_w - ref_l
    inside = -0.5 * beta * (model_diff - ref_diff)
    return {
        "loss": -F.logsigmoid(inside).mean(),
        "raw_model_loss": 0.5 * (win.mean() + lose.mean()),
        "raw_ref_loss": ref_losses.mean(),
        "model_diff": model_diff.mean(),
        "ref_diff": ref_diff.mean(),
        "implicit_acc": (inside > 0).float().mean(),
    }
