"""Rollout layer: collectors, packers, evaluators, family registry and runtime backends."""

from visionrl_b200.rollouts.batch import RolloutBatch, stack_batches

__all__ = ["RolloutBatch", "stack_batches"]
