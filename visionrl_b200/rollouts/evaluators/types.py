"""Signals an evaluator hands to an algorithm (reference: ``vrl/rollouts/evaluators/types.py:9-35``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class SignalBatch:
    """Per-sample (or per-token) quantities of the policy distribution.

    ``log_prob`` is ``[B]`` for diffusion steps and ``[B, L]`` for token policies.
    The flow-matching fields carry what the latent-space KL needs: the Gaussian
    means of policy and reference, the step's ``std_dev_t`` and ``sqrt(-dt)``.
    """

    log_prob: Any
    ref_log_prob: Any | None = None
    entropy: Any | None = None
    prev_sample_mean: Any | None = None
    ref_prev_sample_mean: Any | None = None
    std_dev_t: Any | None = None
    dt: Any | None = None
    dist_family: str = "flow_matching"
    aux: dict[str, Any] = field(default_factory=dict)


@dataclass
class SignalRequest:
    """Which optional signals the algorithm wants computed."""

    need_ref: bool = False
    need_entropy: bool = False
    need_kl_intermediates: bool = False
