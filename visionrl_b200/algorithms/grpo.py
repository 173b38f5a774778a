"""Group-relative policy optimisation on per-sample log-probabilities.

Advantages: for every group of more than one sample,
``a = clamp((r - mean_g) / max(std_g, eps), ±adv_clip_max)`` with the unbiased
group std (or the whole-batch std when ``global_std``); singleton groups get 0.
Loss: ``rho = exp(lp - lp_old)``, ``L = mean(max(-a rho, -a clamp(rho, 1±eps_clip)))``
plus ``init_kl_coef * KL`` where KL is the latent-space Gaussian KL when the
flow-matching means are present and ``mean(lp - lp_ref)`` otherwise
(reference: ``vrl/algorithms/grpo.py:47-161``).  Group statistics are computed
with segment sums — no Python loop over groups.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from visionrl_b200.algorithms.base import Algorithm
from visionrl_b200.algorithms.types import TrainStepMetrics
from visionrl_b200.rollouts.evaluators.types import SignalBatch


@dataclass(slots=True)
class GRPOConfig:
    eps_clip: float = 0.2
    init_kl_coef: float = 0.0
    eps: float = 1e-8
    adv_clip_max: float = 5.0
    global_std: bool = False
    flow_kl_use_dt: bool = False


def group_normalized_advantages(rewards, group_ids, eps: float, adv_clip_max: float,
                                global_std: bool = False):
    """Vectorised group mean/std normalisation (kernel K13's oracle)."""
    import torch

    if rewards.is_cuda and rewards.dim() == 1 and 0 < rewards.numel() <= 16384:
        from visionrl_b200.ops import _ext

        if _ext.kernels_enabled() and _ext.has("group_advantages"):
            adv = _ext.load().group_advantages(rewards.detach(), group_ids, float(eps),
                                               float(adv_clip_max), bool(global_std))
            return adv.to(rewards.dtype)
    return group_normalized_advantages_reference(rewards, group_ids, eps, adv_clip_max, global_std)


def group_normalized_advantages_reference(rewards, group_ids, eps: float, adv_clip_max: float,
                                          global_std: bool = False):
    """Segment-sum restatement in PyTorch (CPU path and oracle of the kernel)."""
    import torch

    rewards_f = rewards.float()
    _, inverse = torch.unique(group_ids, return_inverse=True)
    n_groups = int(inverse.max().item()) + 1 if inverse.numel() else 0
    ones = torch.ones_like(rewards_f)
    count = torch.zeros(n_groups, device=rewards.device).index_add_(0, inverse, ones)
    total = torch.zeros(n_groups, device=rewards.device).index_add_(0, inverse, rewards_f)
    mean = total / count.clamp_min(1)
    centered = rewards_f - mean[inverse]
    if global_std:
        std_all = rewards_f.std() if rewards_f.numel() > 1 else rewards_f.new_zeros(())
        std = std_all.expand(n_groups)
    else:
        sq = torch.zeros(n_groups, device=rewards.device).index_add_(0, inverse, centered**2)
        std = torch.sqrt(sq / (count - 1).clamp_min(1))
    adv = centered / std.clamp_min(eps)[inverse]
    adv = adv.clamp(-adv_clip_max, adv_clip_max)
    adv = torch.where(count[inverse] > 1, adv, torch.zeros_like(adv))
    return adv.to(rewards.dtype)


class GRPO(Algorithm):
    def __init__(self, config: GRPOConfig | None = None) -> None:
        self.config = config or GRPOConfig()
        # Live (graph-attached) pieces of the last loss; the trainer reads them for
        # its policy-vs-KL gradient split and clears them after backward.
        self._last_policy_loss_tensor: Any = None
        self._last_kl_term_tensor: Any = None
        # Detached on-device metric vector of the last call
        # [loss, policy_loss, kl, clip_fraction, approx_kl].
        self.last_metric_tensor: Any = None
        # When False, ``compute_signal_loss`` does not synchronise the device:
        # the returned metrics object holds zeros and the trainer reads
        # ``last_metric_tensor`` once per step instead.
        self.sync_metrics: bool = True

    def compute_advantages_from_tensors(self, rewards: Any, group_ids: Any) -> Any:
        cfg = self.config
        return group_normalized_advantages(
            rewards, group_ids, cfg.eps, cfg.adv_clip_max, cfg.global_std
        )

    def _kl_term(self, signals: SignalBatch):
        import torch

        from visionrl_b200.algorithms.flow_matching import compute_kl_divergence

        cfg = self.config
        if signals.ref_log_prob is None:
            raise RuntimeError(
                f"GRPOConfig.init_kl_coef={cfg.init_kl_coef} > 0 but signals.ref_log_prob is "
                "None: pass a reference model to the trainer and request need_ref=True."
            )
        if (signals.dist_family == "flow_matching" and signals.prev_sample_mean is not None
                and signals.ref_prev_sample_mean is not None):
            kl = compute_kl_divergence(
                signals.prev_sample_mean, signals.ref_prev_sample_mean, signals.std_dev_t,
                dt=signals.dt if cfg.flow_kl_use_dt else None,
            )
            return torch.mean(kl)
        return torch.mean(signals.log_prob - signals.ref_log_prob)

    def compute_signal_loss(self, signals, advantages, old_log_probs):
        import torch

        from visionrl_b200.ops.losses import grpo_clipped_loss

        cfg = self.config
        policy_loss, clip_fraction, approx_kl = grpo_clipped_loss(
            signals.log_prob, old_log_probs, advantages, cfg.eps_clip
        )
        if cfg.init_kl_coef > 0:
            kl_loss = self._kl_term(signals)
            kl_term = cfg.init_kl_coef * kl_loss
            loss = policy_loss + kl_term
            self._last_kl_term_tensor = kl_term
        else:
            kl_loss = torch.zeros((), device=signals.log_prob.device)
            loss = policy_loss
            self._last_kl_term_tensor = None
        self._last_policy_loss_tensor = policy_loss
        self.last_metric_tensor = torch.stack([
            loss.detach().float(), policy_loss.detach().float(), kl_loss.detach().float(),
            clip_fraction.float(), approx_kl.float(),
        ])
        return loss, self._metrics()

    def _metrics(self) -> TrainStepMetrics:
        if not self.sync_metrics:
            return TrainStepMetrics()
        vals = self.last_metric_tensor.tolist()
        return TrainStepMetrics(loss=vals[0], policy_loss=vals[1], kl_penalty=vals[2],
                                clip_fraction=vals[3], approx_kl=vals[4])
