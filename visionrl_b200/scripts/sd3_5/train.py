"""SD3.5 GRPO recipe (reference: ``vrl/scripts/sd3_5/train.py:29-290``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.scripts.common import (
    build_diffusion_parts, build_reward, diffusion_collector_kwargs, run_online_recipe, setup_run,
)


async def train_sd3_5_grpo(cfg: Any) -> Any:
    from visionrl_b200.models.families.sd3_5.builder import build_sd3_5_runtime_bundle_from_cfg
    from visionrl_b200.rollouts.collector import SD3_5CollectorConfig

    ctx = setup_run(cfg)
    bundle = build_sd3_5_runtime_bundle_from_cfg(cfg, ctx.device, ctx.weight_dtype)
    bundle.metadata["family"] = "sd3_5"
    reward_fn, weights = build_reward(ctx)
    collector_config = SD3_5CollectorConfig(
        max_sequence_length=int(getattr(cfg.sampling, "max_sequence_length", 128)),
        **diffusion_collector_kwargs(cfg))
    parts = build_diffusion_parts(ctx, "sd3_5", bundle, collector_config)
    return await run_online_recipe(ctx, parts, reward_fn, list(weights))
