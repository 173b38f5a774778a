"""Packers: engine outputs → trainer batches."""

from visionrl_b200.rollouts.packers.ar_continuous import ARContinuousRolloutPacker
from visionrl_b200.rollouts.packers.ar_discrete import ARDiscreteRolloutPacker
from visionrl_b200.rollouts.packers.base import RolloutPackContext, RolloutPacker
from visionrl_b200.rollouts.packers.diffusion import DiffusionRolloutPacker

__all__ = ["ARContinuousRolloutPacker", "ARDiscreteRolloutPacker", "DiffusionRolloutPacker",
           "RolloutPackContext", "RolloutPacker"]
