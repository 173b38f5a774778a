"""Flow-matching evaluator: ``model.replay_forward`` → SDE step with the recorded
next latent as ``prev_sample`` → log-prob, Gaussian mean and step scales.  The
reference pass runs without grad; when the reference *is* the policy (LoRA) it
runs inside ``disable_adapter()`` (reference:
``vrl/rollouts/evaluators/diffusion/flow_matching.py:17-119``)."""

from __future__ import annotations

import contextlib
from typing import Any

from visionrl_b200.algorithms import flow_matching as flow_matching_math
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.evaluators.types import SignalBatch, SignalRequest


class FlowMatchingEvaluator:
    def __init__(self, scheduler: Any, noise_level: float = 1.0, sde_type: str = "sde") -> None:
        self.scheduler = scheduler
        self.noise_level = noise_level
        self.sde_type = sde_type

    def _step(self, policy: Any, batch: RolloutBatch, idx: int, t, need_dt: bool):
        noise_pred = policy.replay_forward(batch, idx)["noise_pred"]
        return flow_matching_math.sde_step_with_logprob(
            self.scheduler, noise_pred, t, batch.observations[:, idx],
            prev_sample=batch.actions[:, idx], return_dt=need_dt,
            noise_level=self.noise_level, sde_type=self.sde_type,
        )

    def evaluate(self, model: Any, batch: RolloutBatch, timestep_idx: int,
                 ref_model: Any | None = None,
                 signal_request: SignalRequest | None = None) -> SignalBatch:
        import torch

        req = signal_request or SignalRequest()
        ts = batch.extras["timesteps"]
        t = ts[:, timestep_idx] if ts.ndim > 1 else ts
        res = self._step(model, batch, timestep_idx, t, req.need_kl_intermediates)
        ref = None
        if req.need_ref and ref_model is not None:
            same = ref_model is model and hasattr(model, "disable_adapter")
            with torch.no_grad(), (model.disable_adapter() if same else contextlib.nullcontext()):
                ref = self._step(ref_model, batch, timestep_idx, t, req.need_kl_intermediates)
        return SignalBatch(
            log_prob=res.log_prob,
            ref_log_prob=None if ref is None else ref.log_prob,
            prev_sample_mean=res.prev_sample_mean,
            ref_prev_sample_mean=None if ref is None else ref.prev_sample_mean,
            std_dev_t=res.std_dev_t,
            dt=res.dt if res.dt is not None else (None if ref is None else ref.dt),
            dist_family="flow_matching",
        )


__all__ = ["FlowMatchingEvaluator"]
