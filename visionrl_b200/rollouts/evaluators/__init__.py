"""Evaluators and their signal types."""

from visionrl_b200.rollouts.evaluators.base import Evaluator
from visionrl_b200.rollouts.evaluators.types import SignalBatch, SignalRequest

__all__ = ["Evaluator", "SignalBatch", "SignalRequest"]
