"""Per-token GRPO for autoregressive policies.

Sequence-level advantages ``[B]`` are broadcast over ``[B, L]`` tokens; the
clipped surrogate is averaged with a mask, ``sum(loss*m) / max(sum(m), 1)``; the
KL penalty uses ``k1 = d`` or ``k3 = exp(d)(d-1)+1`` with ``d = lp - lp_ref`` and is
applied only when ``init_kl_coef > 0`` and a reference log-prob is present
(reference: ``vrl/algorithms/grpo_token.py:33-158``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from visionrl_b200.algorithms.grpo import GRPO, GRPOConfig
from visionrl_b200.rollouts.evaluators.types import SignalBatch


@dataclass(slots=True)
class TokenGRPOConfig(GRPOConfig):
    mask_key: str = "token_mask"
    kl_estimator: str = "k3"


class TokenGRPO(GRPO):
    def __init__(self, config: TokenGRPOConfig | None = None) -> None:
        cfg = config or TokenGRPOConfig()
        super().__init__(cfg)
        self.config: TokenGRPOConfig = cfg

    def compute_signal_loss(self, signals: SignalBatch, advantages: Any, old_log_probs: Any):
        import torch

        from visionrl_b200.ops.losses import token_grpo_loss

        cfg = self.config
        new_lp = signals.log_prob
        if new_lp.shape != old_log_probs.shape:
            raise ValueError(
                f"log_prob shape mismatch: new={tuple(new_lp.shape)} "
                f"old={tuple(old_log_probs.shape)}"
            )
        if cfg.kl_estimator not in ("k1", "k3"):
            raise ValueError(f"unknown kl_estimator: {cfg.kl_estimator}")
        mask = signals.aux.get(cfg.mask_key) if signals.aux else None
        ref_lp = signals.ref_log_prob if cfg.init_kl_coef > 0 else None
        policy_loss, kl_loss, clip_fraction, approx_kl = token_grpo_loss(
            new_lp, old_log_probs, advantages, mask, ref_lp, cfg.eps_clip, cfg.kl_estimator
        )
        loss = policy_loss + cfg.init_kl_coef * kl_loss if ref_lp is not None else policy_loss
        self._last_policy_loss_tensor = policy_loss
        self._last_kl_term_tensor = cfg.init_kl_coef * kl_loss if ref_lp is not None else None
        self.last_metric_tensor = torch.stack([
            loss.detach().float(), policy_loss.detach().float(), kl_loss.detach().float(),
            clip_fraction.float(), approx_kl.float(),
        ])
        return loss, self._metrics()
