"""Packer protocol: engine ``OutputBatch`` + rewards → ``RolloutBatch``
(reference: ``vrl/rollouts/packers/base.py:12-43``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol

from visionrl_b200.engine import OutputBatch
from visionrl_b200.rollouts.batch import RolloutBatch


@dataclass(slots=True)
class RolloutPackContext:
    metadata: dict[str, Any]
    device: Any | None = None
    kl_reward: float = 0.0
    rescale_to_unit: bool = False
    extra: dict[str, Any] = field(default_factory=dict)


class RolloutPacker(Protocol):
    def reward_outputs(self, output: OutputBatch, context: RolloutPackContext) -> Any: ...
    def reward_prompts(self, output: OutputBatch, context: RolloutPackContext) -> list[str]: ...
    async def pack(self, output: OutputBatch, rewards_raw: Any,
                   context: RolloutPackContext) -> RolloutBatch: ...


def prompt_group_ids(output: OutputBatch, device):
    import torch

    return torch.tensor([s.prompt_index for s in output.sample_specs], dtype=torch.long,
                        device=device)


__all__ = ["RolloutPackContext", "RolloutPacker", "prompt_group_ids"]
