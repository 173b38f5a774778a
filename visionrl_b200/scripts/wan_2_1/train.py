"""Wan-2.1 GRPO recipe (1.3B and 14B shapes) (reference: ``vrl/scripts/wan_2_1/train.py:31-296``).
With ``distributed.mesh.sp > 1`` the transformer runs Ulysses sequence-parallel."""

from __future__ import annotations

from typing import Any

from visionrl_b200.scripts.common import (
    build_diffusion_parts, build_reward, diffusion_collector_kwargs, run_online_recipe, setup_run,
)


async def train_wan_2_1_grpo(cfg: Any) -> Any:
    from visionrl_b200.models.families.wan_2_1.builder import build_wan_2_1_runtime_bundle_from_cfg
    from visionrl_b200.rollouts.collector import Wan_2_1CollectorConfig

    ctx = setup_run(cfg)
    bundle = build_wan_2_1_runtime_bundle_from_cfg(cfg, ctx.device, ctx.weight_dtype)
    bundle.metadata["family"] = "wan_2_1"
    if ctx.mesh.sp > 1:
        from visionrl_b200.parallel.ulysses import attach_sequence_parallel

        attach_sequence_parallel(bundle.policy, ctx.mesh)
    reward_fn, weights = build_reward(ctx)
    collector_config = Wan_2_1CollectorConfig(
        num_frames=int(cfg.sampling.num_frames),
        max_sequence_length=int(getattr(cfg.sampling, "max_sequence_length", 512)),
        **diffusion_collector_kwargs(cfg))
    parts = build_diffusion_parts(ctx, "wan_2_1", bundle, collector_config)
    return await run_online_recipe(ctx, parts, reward_fn, list(weights))
