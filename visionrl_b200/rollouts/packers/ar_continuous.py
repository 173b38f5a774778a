"""Packer for continuous-token rollouts: actions are the tokens ``[B, L, D]`` and the
saved last-step noise rides along for exact log-prob replay
(reference: ``vrl/rollouts/packers/ar_continuous.py:14-75``)."""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.engine import OutputBatch
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.packers.ar_discrete import _unit_images
from visionrl_b200.rollouts.packers.base import RolloutPackContext, prompt_group_ids


class ARContinuousRolloutPacker:
    def reward_outputs(self, output: OutputBatch, context: RolloutPackContext) -> Any:
        ready = output.extra.get("images_for_reward") if isinstance(output.extra, dict) else None
        return ready if ready is not None else _unit_images(output.output, context.rescale_to_unit)

    def reward_prompts(self, output: OutputBatch, context: RolloutPackContext) -> list[str]:
        return [s.prompt for s in output.sample_specs]

    async def pack(self, output: OutputBatch, rewards_raw: torch.Tensor,
                   context: RolloutPackContext) -> RolloutBatch:
        ex = output.extra
        device = context.device or ex["prompt_input_ids"].device
        n = len(output.sample_specs)
        old = ex["log_probs"]
        return RolloutBatch(
            observations=ex["prompt_input_ids"].unsqueeze(1), actions=ex["tokens"],
            rewards=rewards_raw.to(device), dones=torch.ones(n, dtype=torch.bool, device=device),
            group_ids=prompt_group_ids(output, device),
            extras={"log_probs": old.detach().unsqueeze(1),
                    "prompt_attention_mask": ex["prompt_attention_mask"],
                    "uncond_input_ids": ex["uncond_input_ids"],
                    "uncond_attention_mask": ex["uncond_attention_mask"],
                    "token_mask": torch.ones_like(old), "saved_noise": ex["saved_noise"]},
            context=dict(ex["context"]), videos=output.output.unsqueeze(2),
            prompts=[s.prompt for s in output.sample_specs],
        )


__all__ = ["ARContinuousRolloutPacker"]
