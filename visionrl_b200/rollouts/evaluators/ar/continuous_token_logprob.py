"""Evaluator for continuous-token policies: ``replay_forward`` already returns
per-token Gaussian log-probs recomputed with the saved rollout noise
(reference: ``vrl/rollouts/evaluators/ar/continuous_token_logprob.py:24-94``)."""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.evaluators.ar.token_logprob import _has_active_adapter
from visionrl_b200.rollouts.evaluators.types import SignalBatch, SignalRequest


class ContinuousTokenLogProbEvaluator:
    def __init__(self, mask_key: str = "token_mask") -> None:
        self.mask_key = mask_key

    @staticmethod
    def _log_probs(model: Any, batch: RolloutBatch) -> torch.Tensor:
        out = model.replay_forward(batch, timestep_idx=0)
        if "log_probs" not in out:
            raise KeyError("continuous-token replay_forward must return 'log_probs'")
        return out["log_probs"]

    def evaluate(self, model: Any, batch: RolloutBatch, timestep_idx: int = 0,
                 ref_model: Any | None = None,
                 signal_request: SignalRequest | None = None) -> SignalBatch:
        req = signal_request or SignalRequest()
        new_lp = self._log_probs(model, batch)
        ref_lp = None
        if req.need_ref:
            if ref_model is not None and ref_model is not model:
                with torch.no_grad():
                    ref_lp = self._log_probs(ref_model, batch)
            else:
                if not _has_active_adapter(model):
                    raise RuntimeError(
                        "ContinuousTokenLogProbEvaluator: need_ref=True but there is neither an "
                        "adapter to disable nor a ref_model")
                with torch.no_grad(), model.disable_adapter():
                    ref_lp = self._log_probs(model, batch)
        aux = {self.mask_key: batch.extras[self.mask_key]} if self.mask_key in batch.extras else {}
        return SignalBatch(log_prob=new_lp, ref_log_prob=ref_lp, entropy=None,
                           dist_family="continuous_flow", aux=aux)


__all__ = ["ContinuousTokenLogProbEvaluator"]
