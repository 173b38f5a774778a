"""Packer for categorical image-token rollouts: observations are the prompt ids
``[B, 1, L_text]``, actions the sampled tokens ``[B, L_img]``
(reference: ``vrl/rollouts/packers/ar_discrete.py:14-75``)."""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.engine import OutputBatch
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.packers.base import RolloutPackContext, prompt_group_ids


def _unit_images(images, rescale: bool):
    return ((images + 1.0) * 0.5).clamp(0.0, 1.0) if rescale else images


class ARDiscreteRolloutPacker:
    def reward_outputs(self, output: OutputBatch, context: RolloutPackContext) -> Any:
        return _unit_images(output.output, context.rescale_to_unit)

    def reward_prompts(self, output: OutputBatch, context: RolloutPackContext) -> list[str]:
        return [s.prompt for s in output.sample_specs]

    async def pack(self, output: OutputBatch, rewards_raw: torch.Tensor,
                   context: RolloutPackContext) -> RolloutBatch:
        ex = output.extra
        device = context.device or ex["prompt_input_ids"].device
        n = len(output.sample_specs)
        return RolloutBatch(
            observations=ex["prompt_input_ids"].unsqueeze(1), actions=ex["token_ids"],
            rewards=rewards_raw.to(device), dones=torch.ones(n, dtype=torch.bool, device=device),
            group_ids=prompt_group_ids(output, device),
            extras={"log_probs": ex["token_log_probs"].detach().unsqueeze(1),
                    "prompt_attention_mask": ex["prompt_attention_mask"],
                    "uncond_input_ids": ex["uncond_input_ids"],
                    "uncond_attention_mask": ex["uncond_attention_mask"],
                    "token_mask": ex["token_mask"]},
            context=dict(ex.get("context", {})), videos=output.output.unsqueeze(2),
            prompts=[s.prompt for s in output.sample_specs],
        )


__all__ = ["ARDiscreteRolloutPacker"]
