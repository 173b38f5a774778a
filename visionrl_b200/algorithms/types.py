"""Plain data containers shared by algorithms, rewards and trainers
(reference: ``vrl/algorithms/types.py:10-60``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(slots=True)
class TrajectoryStep:
    """One denoising step of a recorded trajectory."""

    timestep: int
    log_prob: Any
    noise_pred: Any
    new_log_prob: Any = None
    ref_log_prob: Any = None


@dataclass(slots=True)
class Trajectory:
    """All steps plus the final artefact (frames or latents) of one sample."""

    prompt: str
    seed: int
    steps: list[TrajectoryStep]
    output: Any


@dataclass(slots=True)
class Rollout:
    """A generated sample as the reward layer sees it."""

    request: Any
    trajectory: Trajectory
    reward: float = 0.0
    metadata: dict[str, Any] = field(default_factory=dict)


@dataclass(slots=True)
class TrainStepMetrics:
    """Scalar metrics of one trainer step (the ``metrics.csv`` schema)."""

    loss: float = 0.0
    policy_loss: float = 0.0
    kl_penalty: float = 0.0
    reward_mean: float = 0.0
    reward_std: float = 0.0
    advantage_mean: float = 0.0
    clip_fraction: float = 0.0
    approx_kl: float = 0.0
    grad_norm: float = 0.0
    adv_saturation: float = 0.0
    adv_zero_rate: float = 0.0
    lr: float = 0.0
    group_size: float = 0.0
    trained_prompt_num: int = 0
    phase_times: dict[str, float] = field(default_factory=dict)
