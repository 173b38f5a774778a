"""Diffusion evaluators."""
from visionrl_b200.rollouts.evaluators.diffusion.flow_matching import FlowMatchingEvaluator

__all__ = ["FlowMatchingEvaluator"]
