"""NextStep-1 TokenGRPO recipe with the OCR reward
(reference: ``vrl/scripts/nextstep_1/train.py:43-306``).  Steps are counted from 1."""

from __future__ import annotations

from typing import Any

from visionrl_b200.scripts.common import RecipeParts, build_reward, run_online_recipe, setup_run

NEXTSTEP_CSV_HEAD = ("step,loss,policy_loss,kl_penalty,reward_mean,reward_std,clip_fraction,approx_kl,"
                     "advantage_mean,grad_norm,adv_saturation,adv_zero_rate,group_size,trained_prompt_num")


async def train_nextstep_1_ocr_grpo(cfg: Any) -> Any:
    from visionrl_b200.algorithms.grpo_token import TokenGRPO, TokenGRPOConfig
    from visionrl_b200.algorithms.stat_tracking import PerPromptStatTracker
    from visionrl_b200.config.loader import require
    from visionrl_b200.models.families.nextstep_1.builder import (
        build_nextstep_1_runtime_bundle_from_cfg,
    )
    from visionrl_b200.rollouts.collector import NextStep1CollectorConfig
    from visionrl_b200.rollouts.evaluators.ar import ContinuousTokenLogProbEvaluator

    ctx = setup_run(cfg)
    algo_cfg = ctx.built["algorithm"]
    if not isinstance(algo_cfg, TokenGRPOConfig):
        raise TypeError(f"NextStep-1 expects algorithm.kind=token_grpo, got {type(algo_cfg).__name__}")
    bundle = build_nextstep_1_runtime_bundle_from_cfg(cfg, ctx.device, ctx.weight_dtype)
    policy = bundle.policy
    if ctx.trainer_config.gradient_checkpointing:
        policy.language_model.gradient_checkpointing = True
    reward_fn, weights = build_reward(ctx)
    collector_config = NextStep1CollectorConfig(
        n_samples_per_prompt=int(require(cfg, "rollout.n_samples_per_prompt")),
        cfg_scale=float(cfg.sampling.cfg_scale), num_flow_steps=int(cfg.sampling.num_flow_steps),
        noise_level=float(require(cfg, "rollout.noise_level")),
        image_token_num=int(cfg.sampling.image_token_num), image_size=int(cfg.sampling.image_size),
        rescale_to_unit=bool(require(cfg, "rollout.rescale_to_unit")),
        max_text_length=int(require(cfg, "rollout.max_text_length")))
    need_ref = algo_cfg.init_kl_coef > 0
    tracker = PerPromptStatTracker(global_std=algo_cfg.global_std) \
        if cfg.algorithm.per_prompt_stat_tracking else None
    parts = RecipeParts(
        family="nextstep_1", bundle=bundle, collector_config=collector_config,
        evaluator=ContinuousTokenLogProbEvaluator(mask_key=algo_cfg.mask_key),
        algorithm=TokenGRPO(algo_cfg), ref_model=policy if need_ref else None,
        stat_tracker=tracker, csv_columns=NEXTSTEP_CSV_HEAD, first_epoch=1,
        adapter_module=policy.language_model)
    return await run_online_recipe(ctx, parts, reward_fn, list(weights))
