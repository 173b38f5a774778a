"""Janus-Pro TokenGRPO recipes (reference: ``vrl/scripts/janus_pro/train.py:48-362``).

Two entry points share one body: ``train_janus_pro_grpo`` (reward mix from the config) and
``train_janus_pro_ocr_grpo`` (OCR reward).  The policy is checkpointed under the trainable
module name ``policy``; the CSV lists ``approx_kl`` before ``clip_fraction``.
"""

from __future__ import annotations

from typing import Any

from visionrl_b200.scripts.common import RecipeParts, build_reward, run_online_recipe, setup_run

JANUS_CSV_HEAD = ("epoch,loss,policy_loss,kl_penalty,reward_mean,reward_std,approx_kl,clip_fraction,"
                  "advantage_mean,grad_norm,adv_saturation,adv_zero_rate,group_size,trained_prompt_num")


def _janus_csv_row(epoch: int, m: Any) -> str:
    return (f"{epoch},{m.loss:.6f},{m.policy_loss:.6f},{m.kl_penalty:.6f},{m.reward_mean:.4f},"
            f"{m.reward_std:.4f},{m.approx_kl:.6f},{m.clip_fraction:.4f},{m.advantage_mean:.6f},"
            f"{m.grad_norm:.6f},{m.adv_saturation:.4f},{m.adv_zero_rate:.4f},{m.group_size:.2f},"
            f"{m.trained_prompt_num}")


async def _train_janus_pro(cfg: Any) -> Any:
    from visionrl_b200.algorithms.grpo_token import TokenGRPO, TokenGRPOConfig
    from visionrl_b200.algorithms.stat_tracking import PerPromptStatTracker
    from visionrl_b200.config.loader import require
    from visionrl_b200.models.families.janus_pro.builder import (
        build_janus_pro_runtime_bundle_from_cfg,
    )
    from visionrl_b200.rollouts.collector import JanusProCollectorConfig
    from visionrl_b200.rollouts.evaluators.ar import TokenLogProbEvaluator

    ctx = setup_run(cfg)
    algo_cfg = ctx.built["algorithm"]
    if not isinstance(algo_cfg, TokenGRPOConfig):
        raise TypeError(f"Janus-Pro expects algorithm.kind=token_grpo, got {type(algo_cfg).__name__}")
    bundle = build_janus_pro_runtime_bundle_from_cfg(cfg, ctx.device, ctx.weight_dtype)
    policy = bundle.policy
    if ctx.trainer_config.gradient_checkpointing:
        policy.language_model.gradient_checkpointing = True
    reward_fn, weights = build_reward(ctx)
    collector_config = JanusProCollectorConfig(
        n_samples_per_prompt=int(require(cfg, "rollout.n_samples_per_prompt")),
        cfg_weight=float(cfg.sampling.cfg_weight),
        temperature=float(getattr(cfg.sampling, "temperature", cfg.rollout.get("temperature", 1.0))),
        image_token_num=int(cfg.sampling.image_token_num), image_size=int(cfg.sampling.image_size),
        rescale_to_unit=bool(require(cfg, "rollout.rescale_to_unit")),
        max_text_length=int(require(cfg, "rollout.max_text_length")))
    need_ref = algo_cfg.init_kl_coef > 0
    if need_ref and not policy.has_adapters:
        raise ValueError("algorithm.init_kl_coef > 0 needs model.use_lora=true (the reference "
                         "policy is the trunk with adapters disabled)")
    tracker = PerPromptStatTracker(global_std=algo_cfg.global_std) \
        if cfg.algorithm.per_prompt_stat_tracking else None
    parts = RecipeParts(
        family="janus_pro", bundle=bundle, collector_config=collector_config,
        evaluator=TokenLogProbEvaluator(mask_key=algo_cfg.mask_key), algorithm=TokenGRPO(algo_cfg),
        ref_model=policy if need_ref else None, stat_tracker=tracker,
        csv_columns=JANUS_CSV_HEAD, csv_row=_janus_csv_row,
        adapter_module=policy.language_model)
    return await run_online_recipe(ctx, parts, reward_fn, list(weights))


async def train_janus_pro_grpo(cfg: Any) -> Any:
    return await _train_janus_pro(cfg)


async def train_janus_pro_ocr_grpo(cfg: Any) -> Any:
    return await _train_janus_pro(cfg)
