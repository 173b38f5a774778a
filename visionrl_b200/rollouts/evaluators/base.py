"""Evaluator protocol: replay a recorded step through the policy and extract the
signals a loss needs (reference: ``vrl/rollouts/evaluators/base.py:11-31``)."""

from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.evaluators.types import SignalBatch, SignalRequest


@runtime_checkable
class Evaluator(Protocol):
    def evaluate(self, model: Any, batch: RolloutBatch, timestep_idx: int,
                 ref_model: Any | None = None,
                 signal_request: SignalRequest | None = None) -> SignalBatch: ...
