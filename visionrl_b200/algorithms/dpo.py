"""Diffusion-DPO objective on winner/loser pairs stacked along the batch axis.

``l = mean_{non-batch}((pred - target)^2)`` is split into winner and loser halves;
``D = l_w - l_l``; ``inside = -beta/2 (D_model - D_ref)``; ``loss = -logsigmoid(inside).mean()``;
``implicit_acc = mean(inside > 0)`` (reference: ``vrl/algorithms/dpo.py:34-114``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass(slots=True)
class DiffusionDPOConfig:
    beta: float = 5000.0
    sft_weight: float = 0.0


def diffusion_dpo_loss(model_pred: torch.Tensor, ref_pred: torch.Tensor, target: torch.Tensor,
                       beta: float) -> dict[str, torch.Tensor]:
    if model_pred.shape != ref_pred.shape or model_pred.shape != target.shape:
        raise ValueError(
            f"shape mismatch: model_pred={tuple(model_pred.shape)} "
            f"ref_pred={tuple(ref_pred.shape)} target={tuple(target.shape)}"
        )
    if model_pred.shape[0] % 2 != 0:
        raise ValueError(f"leading dim must be 2*B (winner-then-loser); got {model_pred.shape[0]}")
    from visionrl_b200.ops.losses import dpo_loss_reference, per_sample_mse

    if model_pred.is_cuda:
        # reference branch: fused per-sample MSE kernel, no autograd graph needed
        with torch.no_grad():
            ref_losses = per_sample_mse(ref_pred.detach(), target.detach())
        dims = tuple(range(1, model_pred.ndim))
        model_losses = (model_pred.float() - target.float()).pow(2).mean(dim=dims)
        win, lose = model_losses.chunk(2)
        ref_w, ref_l = ref_losses.chunk(2)
        model_diff, ref_diff = win - lose, ref_w - ref_l
        inside = -0.5 * beta * (model_diff - ref_diff)
        return {
            "loss": -F.logsigmoid(inside).mean(),
            "raw_model_loss": 0.5 * (win.mean() + lose.mean()),
            "raw_ref_loss": ref_losses.mean(),
            "model_diff": model_diff.mean(),
            "ref_diff": ref_diff.mean(),
            "implicit_acc": (inside > 0).float().mean(),
        }
    return dpo_loss_reference(model_pred, ref_pred, target, beta)


def diffusion_sft_loss(model_pred_winner: torch.Tensor, target_winner: torch.Tensor) -> torch.Tensor:
    """MSE on the winner half only."""
    return F.mse_loss(model_pred_winner.float(), target_winner.float(), reduction="mean")


__all__ = ["DiffusionDPOConfig", "diffusion_dpo_loss", "diffusion_sft_loss"]
