"""Advantage estimation and policy losses."""

from visionrl_b200.algorithms.base import Algorithm
from visionrl_b200.algorithms.flow_matching import (
    SDEStepResult,
    compute_kl_divergence,
    sde_step_with_logprob,
)
from visionrl_b200.algorithms.grpo import GRPO, GRPOConfig
from visionrl_b200.algorithms.types import Rollout, TrainStepMetrics, Trajectory, TrajectoryStep

__all__ = [
    "GRPO", "Algorithm", "GRPOConfig", "Rollout", "SDEStepResult", "TrainStepMetrics",
    "Trajectory", "TrajectoryStep", "compute_kl_divergence", "sde_step_with_logprob",
]
