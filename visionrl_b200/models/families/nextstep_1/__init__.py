"""nextstep_1 model family."""
from visionrl_b200.models.families.nextstep_1.policy import NextStep1Config, NextStep1Policy

__all__ = ["NextStep1Config", "NextStep1Policy"]
