"""Algorithm interface of the collector → evaluator → algorithm loop
(reference: ``vrl/algorithms/base.py:12-35``)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any

from visionrl_b200.algorithms.types import TrainStepMetrics
from visionrl_b200.rollouts.evaluators.types import SignalBatch


class Algorithm(ABC):
    @abstractmethod
    def compute_advantages_from_tensors(self, rewards: Any, group_ids: Any) -> Any:
        """``rewards[B]``, ``group_ids[B]`` → ``advantages[B]``."""

    @abstractmethod
    def compute_signal_loss(
        self, signals: SignalBatch, advantages: Any, old_log_probs: Any
    ) -> tuple[Any, TrainStepMetrics]:
        """Loss tensor (with graph) and detached metrics."""
