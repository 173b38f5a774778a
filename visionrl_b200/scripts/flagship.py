"""Programmatic construction of the SD3.5-shape GRPO trainer (the flagship workload).

``build_flagship_trainer(cfg)`` performs exactly what the ``train_sd3_5_grpo`` recipe does up
to the epoch loop and returns ``(trainer, prompts)``, so benchmarks and smoke tests drive the
same public objects a training run uses (``OnlineTrainer.step``).
"""

from __future__ import annotations

from typing import Any

import torch

from visionrl_b200.scripts.common import (
    build_diffusion_parts, build_online_trainer, build_reward, diffusion_collector_kwargs,
    setup_run,
)


def build_flagship_trainer(cfg: Any, num_prompts: int | None = None):
    from visionrl_b200.config.loader import require
    from visionrl_b200.models.families.sd3_5.builder import build_sd3_5_runtime_bundle_from_cfg
    from visionrl_b200.rollouts.collector import SD3_5CollectorConfig
    from visionrl_b200.trainers.data import load_prompt_manifest

    ctx = setup_run(cfg)
    bundle = build_sd3_5_runtime_bundle_from_cfg(cfg, ctx.device, ctx.weight_dtype)
    bundle.metadata["family"] = "sd3_5"
    reward_fn, _ = build_reward(ctx)
    collector_config = SD3_5CollectorConfig(
        max_sequence_length=int(getattr(cfg.sampling, "max_sequence_length", 128)),
        **diffusion_collector_kwargs(cfg))
    parts = build_diffusion_parts(ctx, "sd3_5", bundle, collector_config)
    trainer, _ = build_online_trainer(ctx, parts, reward_fn)
    examples = load_prompt_manifest(str(require(cfg, "data.manifest")))
    count = num_prompts if num_prompts is not None else ctx.trainer_config.rollout_batch_size
    gen = torch.Generator().manual_seed(ctx.trainer_config.seed)
    picked = torch.randperm(len(examples), generator=gen)[:count].tolist()
    return trainer, [examples[i] for i in picked]
