"""Autoregressive evaluators."""
from visionrl_b200.rollouts.evaluators.ar.continuous_token_logprob import (
    ContinuousTokenLogProbEvaluator,
)
from visionrl_b200.rollouts.evaluators.ar.token_logprob import TokenLogProbEvaluator

__all__ = ["ContinuousTokenLogProbEvaluator", "TokenLogProbEvaluator"]
