"""Per-token log-prob evaluator for categorical image-token policies.

The policy's ``replay_forward`` returns either ``{"logits"}`` (``[B, L, V]``) or,
on the fused path, ``{"token_log_probs"}`` computed by the gen-head GEMM +
log-softmax + gather kernel without materialising fp32 logits.  Logits are
divided by the rollout temperature recorded in ``batch.context`` before the
softmax.  With ``need_ref`` the reference comes from ``ref_model`` or from the
same model with adapters disabled; if neither exists the call raises instead of
returning ``ref == policy`` (reference:
``vrl/rollouts/evaluators/ar/token_logprob.py:25-122``).
"""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.ops.logprob import token_log_probs
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.evaluators.types import SignalBatch, SignalRequest


def _has_active_adapter(model: Any) -> bool:
    flag = getattr(model, "has_adapters", None)
    if flag is not None:
        return bool(flag)
    sub = getattr(model, "language_model", None) or model
    return callable(getattr(sub, "disable_adapter", None))


class TokenLogProbEvaluator:
    def __init__(self, mask_key: str = "token_mask") -> None:
        self.mask_key = mask_key

    @staticmethod
    def _compute_logprobs(model: Any, batch: RolloutBatch, action_ids: torch.Tensor) -> torch.Tensor:
        out = model.replay_forward(batch, timestep_idx=0)
        if "token_log_probs" in out:
            return out["token_log_probs"]
        temperature = float((batch.context or {}).get("temperature", 1.0) or 1.0)
        return token_log_probs(out["logits"], action_ids, temperature)

    def evaluate(self, model: Any, batch: RolloutBatch, timestep_idx: int = 0,
                 ref_model: Any | None = None,
                 signal_request: SignalRequest | None = None) -> SignalBatch:
        req = signal_request or SignalRequest()
        ids = batch.actions
        new_lp = self._compute_logprobs(model, batch, ids)
        ref_lp = None
        if req.need_ref:
            if ref_model is not None and ref_model is not model:
                with torch.no_grad():
                    ref_lp = self._compute_logprobs(ref_model, batch, ids)
            else:
                if not _has_active_adapter(model):
                    raise RuntimeError(
                        "TokenLogProbEvaluator: need_ref=True but the model has no adapter to "
                        "disable and no ref_model was provided; ref_log_prob would equal "
                        "log_prob and the KL penalty would be identically zero."
                    )
                with torch.no_grad(), model.disable_adapter():
                    ref_lp = self._compute_logprobs(model, batch, ids)
        aux = {self.mask_key: batch.extras[self.mask_key]} if self.mask_key in batch.extras else {}
        return SignalBatch(log_prob=new_lp, ref_log_prob=ref_lp, entropy=None,
                           dist_family="categorical", aux=aux)


__all__ = ["TokenLogProbEvaluator"]
