"""Diffusion packer: latent trajectory, per-step log-probs, timesteps and replay
conditioning (reference: ``vrl/rollouts/packers/diffusion.py:14-107``).  With
``kl_reward > 0`` the reward is shaped by ``- kl_reward * sum_t kl_t``."""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.engine import OutputBatch
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.packers.base import RolloutPackContext, prompt_group_ids


class DiffusionRolloutPacker:
    def __init__(self, *, error_prefix: str) -> None:
        self.error_prefix = error_prefix

    def _env(self, output: OutputBatch) -> dict[str, Any]:
        rt = output.rollout_trajectory_data
        if rt is None or rt.denoising_env is None:
            raise RuntimeError(f"{self.error_prefix} OutputBatch is missing denoising_env")
        return rt.denoising_env.extra

    def reward_outputs(self, output: OutputBatch, context: RolloutPackContext) -> Any:
        return self._env(output)["videos"]

    def reward_prompts(self, output: OutputBatch, context: RolloutPackContext) -> list[str]:
        return [s.prompt for s in output.sample_specs]

    async def pack(self, output: OutputBatch, rewards_raw: torch.Tensor,
                   context: RolloutPackContext) -> RolloutBatch:
        rt = output.rollout_trajectory_data
        if rt is None or rt.dit_trajectory is None:
            raise RuntimeError(
                f"{self.error_prefix} OutputBatch is missing rollout_trajectory_data / dit_trajectory")
        env = self._env(output)
        obs, actions, log_probs = rt.dit_trajectory.latents, env["actions"], rt.rollout_log_probs
        if obs is None or actions is None or log_probs is None:
            raise RuntimeError(f"{self.error_prefix} OutputBatch is missing trajectory tensors "
                               "(observations/actions/log_probs)")
        n, device = obs.shape[0], obs.device
        if len(output.sample_specs) != n:
            raise RuntimeError(
                f"{self.error_prefix} OutputBatch sample_specs length does not match batch size")
        raw = rewards_raw.to(device)
        shaped = raw - context.kl_reward * env["kl"].sum(dim=1) if context.kl_reward > 0 else raw
        extras = {"log_probs": log_probs, "timesteps": rt.dit_trajectory.timesteps,
                  "kl": env["kl"], "reward_before_kl": raw, **env["training_extras"]}
        return RolloutBatch(
            observations=obs, actions=actions, rewards=shaped,
            dones=torch.ones(n, dtype=torch.bool, device=device),
            group_ids=prompt_group_ids(output, device), extras=extras, context=env["context"],
            videos=env["videos"], prompts=[s.prompt for s in output.sample_specs],
        )


__all__ = ["DiffusionRolloutPacker"]
