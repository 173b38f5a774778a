"""Reward functions."""

from typing import Any

from visionrl_b200.rewards.base import RewardFunction
from visionrl_b200.rewards.composite import CompositeReward
from visionrl_b200.rewards.multi import MultiReward, get_reward, register_reward


def __getattr__(name: str) -> Any:
    if name == "RemoteReward":
        from visionrl_b200.rewards.remote import RemoteReward

        return RemoteReward
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["CompositeReward", "MultiReward", "RemoteReward", "RewardFunction", "get_reward",
           "register_reward"]
