"""Cosmos-Predict2 GRPO recipe (reference: ``vrl/scripts/cosmos/train.py:32-557``).

Adds to the common loop: the reference image, epoch-0 sanity gates on ``clip_fraction`` /
``approx_kl``, evaluation sample dumps at checkpoints and an eval-only mode that compares the
adapter against the base model on fixed prompts and seeds without training.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

import torch

from visionrl_b200.rollouts.runtime.config import cfg_path
from visionrl_b200.scripts.common import (
    CSV_HEAD, build_diffusion_parts, build_online_trainer, build_reward, default_csv_row,
    diffusion_collector_kwargs, run_online_recipe, setup_run,
)

logger = logging.getLogger(__name__)


def save_eval_frames(videos: torch.Tensor, out_dir: Path, tag: str) -> list[Path]:
    """Middle frame of every ``[3, T, H, W]`` video in ``[0, 1]`` → ``<tag>.png`` for a single
    video, ``<tag>_<i>.png`` for several."""
    from PIL import Image

    out_dir.mkdir(parents=True, exist_ok=True)
    paths = []
    for i, video in enumerate(videos):
        frame = video[:, video.shape[1] // 2] if video.ndim == 4 else video
        arr = (frame.clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
        path = out_dir / (f"{tag}.png" if len(videos) == 1 else f"{tag}_{i:03d}.png")
        Image.fromarray(arr).save(path)
        paths.append(path)
    return paths


async def _eval_only(ctx, parts, reward_fn, cfg) -> dict[str, Any]:
    """Paired adapter-vs-base comparison on the eval prompts, the same seeds for both, no training
    (reference: ``vrl/scripts/cosmos/train.py:445-557``).  Writes ``eval_only/eval_results.csv``
    (``prompt, seed, lora_score, base_score, delta``) and the middle frame of every video.

    The rollout workers hold their own copy of the policy, so the base pass does not flip a flag
    on the trainer's module: it zeroes the adapters' ``B`` factors, pushes that state to the
    workers, evaluates, then restores and pushes the trained state again."""
    import csv

    from visionrl_b200.models.nn.layers import adapters_zeroed
    from visionrl_b200.trainers.data import load_prompt_manifest

    lora_path = str(cfg_path(cfg, "model.lora.path", "") or "")
    if not lora_path:
        raise ValueError("eval.eval_only=true requires model.lora.path (a trained adapter)")
    trainer, collector = build_online_trainer(ctx, parts, reward_fn)
    prompts = [e.prompt for e in load_prompt_manifest(str(cfg.eval.prompts_file))]
    seeds = int(cfg.eval.seeds)
    policy = parts.bundle.policy
    out_dir = Path(ctx.trainer_config.output_dir) / "eval_only"
    out_dir.mkdir(parents=True, exist_ok=True)

    async def sweep(tag: str) -> list[float]:
        scores = []
        for p_idx, prompt in enumerate(prompts):
            for seed in range(seeds):
                with torch.no_grad():
                    batch = await collector.collect([prompt], group_size=1, seed=seed)
                score = float(batch.rewards[0])
                scores.append(score)
                if batch.videos is not None:
                    save_eval_frames(batch.videos[:1], out_dir,
                                     f"{tag}_prompt_{p_idx}_seed_{seed}_score_{score:.2f}")
        return scores

    await trainer.push_rollout_weights()
    lora_scores = await sweep("lora")
    with adapters_zeroed(policy.transformer):
        await trainer.push_rollout_weights()
        base_scores = await sweep("base")
    await trainer.push_rollout_weights()

    keys = [(p, s) for p in prompts for s in range(seeds)]
    with open(out_dir / "eval_results.csv", "w", newline="") as fh:
        writer = csv.DictWriter(fh, fieldnames=["prompt", "seed", "lora_score", "base_score", "delta"])
        writer.writeheader()
        for (prompt, seed), lo, ba in zip(keys, lora_scores, base_scores):
            writer.writerow({"prompt": prompt, "seed": seed, "lora_score": f"{lo:.4f}",
                             "base_score": f"{ba:.4f}", "delta": f"{lo - ba:.4f}"})
    mean = lambda xs: sum(xs) / max(len(xs), 1)  # noqa: E731
    logger.info("Eval-only results: lora=%.4f base=%.4f delta=%.4f | %s", mean(lora_scores),
                mean(base_scores), mean(lora_scores) - mean(base_scores), out_dir / "eval_results.csv")
    shutdown = getattr(collector, "shutdown", None)
    if callable(shutdown):
        await shutdown()
    return {"adapter": lora_scores, "base": base_scores}


async def train_cosmos_predict2_grpo(cfg: Any) -> Any:
    from visionrl_b200.models.families.cosmos.builder import (
        build_cosmos_predict2_runtime_bundle_from_cfg,
    )
    from visionrl_b200.rollouts.collector import CosmosPredict2CollectorConfig

    ctx = setup_run(cfg)
    bundle = build_cosmos_predict2_runtime_bundle_from_cfg(cfg, ctx.device, ctx.weight_dtype)
    bundle.metadata["family"] = "cosmos"
    reward_fn, weights = build_reward(ctx)
    collector_config = CosmosPredict2CollectorConfig(
        num_frames=int(cfg.sampling.num_frames), fps=int(cfg.sampling.fps),
        max_sequence_length=int(getattr(cfg.sampling, "max_sequence_length", 512)),
        **diffusion_collector_kwargs(cfg))
    ref_image = str(cfg_path(cfg, "model.reference_image", "") or "")
    parts = build_diffusion_parts(
        ctx, "cosmos", bundle, collector_config, reference_image=ref_image or None,
        csv_columns=CSV_HEAD + ",ref_image",
        csv_row=lambda epoch, m: default_csv_row(epoch, m) + f",{ref_image or 'none'}")
    if bool(cfg_path(cfg, "eval.eval_only", False)):
        return await _eval_only(ctx, parts, reward_fn, cfg)

    gates = cfg_path(cfg, "eval.sanity_gates", None)

    def on_epoch_end(epoch: int, metrics: Any, trainer: Any) -> None:
        if epoch != 0 or gates is None or not bool(gates.enable):
            return
        if metrics.clip_fraction > float(gates.clip_fraction_threshold):
            raise RuntimeError(
                f"epoch-0 sanity gate: clip_fraction={metrics.clip_fraction:.3f} exceeds "
                f"{float(gates.clip_fraction_threshold)} — rollout and replay log-probs disagree")
        if metrics.approx_kl > float(gates.approx_kl_threshold):
            raise RuntimeError(
                f"epoch-0 sanity gate: approx_kl={metrics.approx_kl:.4f} exceeds "
                f"{float(gates.approx_kl_threshold)}")

    async def on_checkpoint(directory: Path, completed: int, trainer: Any, collector: Any) -> None:
        """One sample per evaluation prompt (seed = its index) beside every periodic checkpoint:
        ``<checkpoint>/eval_samples/prompt_<i>_score_<reward>.png``.  The prompts come from
        ``eval.prompts_file`` when that file exists, else the first four training prompts
        (reference: ``vrl/scripts/cosmos/train.py:210-219,369-398``)."""
        prompts = _eval_prompts(cfg)
        await trainer.push_rollout_weights()
        scores = []
        for i, prompt in enumerate(prompts):
            with torch.no_grad():
                batch = await collector.collect([prompt], group_size=1, seed=i)
            score = float(batch.rewards[0])
            scores.append(score)
            if batch.videos is not None and ctx.mesh.is_main:
                save_eval_frames(batch.videos[:1], directory / "eval_samples", f"prompt_{i}_score_{score:.2f}")
        if ctx.mesh.is_main:
            logger.info("Checkpoint %d | eval_reward=%.4f (%s) | saved to %s", completed,
                        sum(scores) / max(len(scores), 1), ", ".join(f"{s:.2f}" for s in scores), directory)

    dump = bool(cfg_path(cfg, "eval.samples_at_checkpoints", True))
    return await run_online_recipe(ctx, parts, reward_fn, list(weights), on_epoch_end=on_epoch_end,
                                   on_checkpoint=on_checkpoint if dump else None)


def _eval_prompts(cfg: Any) -> list[str]:
    from visionrl_b200.trainers.data import load_prompt_manifest

    held_out = str(cfg_path(cfg, "eval.prompts_file", "") or "")
    if held_out and Path(held_out).exists():
        prompts = [e.prompt for e in load_prompt_manifest(held_out)]
        if prompts:
            return prompts
    return [e.prompt for e in load_prompt_manifest(str(cfg.data.manifest))[:4]]
