"""Wan-2.1 offline Diffusion-DPO recipe (reference: ``vrl/scripts/wan_2_1/train_dpo.py:34-310``).

Preference pairs come from Pick-a-Pic (pixels → latents through the encoder returned by
``_build_encoders``) or, with ``data.dataset_name: synthetic``, from seed-generated latent
pairs.  The learning rate is scaled by the effective batch (accumulation x batch x world) when
``actor.scale_lr`` is set.  The loop writes ``metrics.csv`` and periodic / final checkpoints.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

import torch

from visionrl_b200.config.loader import build_configs, optional_none, require
from visionrl_b200.rollouts.runtime.config import cfg_path
from visionrl_b200.trainers.checkpointing import (
    capture_rng_state, join_trainable_state_gathers, load_training_checkpoint_from_config, prepare_metrics_csv,
    prepare_model_config_for_training_resume, restore_rng_state, restore_training_checkpoint,
    save_resolved_config, save_training_checkpoint,
)

logger = logging.getLogger(__name__)

DPO_CSV_HEAD = "step,loss,raw_model_loss,raw_ref_loss,model_diff,ref_diff,implicit_acc,sft_loss,grad_norm,lr\n"


def _build_encoders(policy: Any, num_frames: int, device: torch.device, dtype: torch.dtype):
    """``(encode_pixels, encode_text)``.

    ``encode_pixels`` maps ``[2B, 3, H, W]`` images in ``[-1, 1]`` to normalised video latents
    ``[2B, C, F', h, w]`` (frames replicated ``num_frames`` times before temporal compression).
    Without an encoder checkpoint the spatial compression is an 8x8 area pooling followed by a
    fixed seeded 3→C channel projection.  ``encode_text`` returns one context row per caption,
    repeated for the winner and loser halves.
    """
    arch = policy.arch
    channels = int(arch["in_channels"])
    scale = int(arch.get("vae_scale", 8))
    t_scale = int(arch.get("vae_temporal_scale", 4))
    gen = torch.Generator().manual_seed(20240)
    proj = (torch.randn(channels, 3, generator=gen) / 3**0.5).to(device)
    decoder = getattr(policy.backend_handle, "decoder", None)
    mean = getattr(decoder, "latents_mean", torch.zeros(channels)).to(device).view(1, channels, 1, 1, 1)
    std = getattr(decoder, "latents_std", torch.ones(channels)).to(device).view(1, channels, 1, 1, 1)
    latent_frames = (num_frames - 1) // t_scale + 1

    def encode_pixels(pixels: torch.Tensor) -> torch.Tensor:
        x = torch.nn.functional.avg_pool2d(pixels.float().to(device), scale)
        z = torch.einsum("cd,bdhw->bchw", proj, x).unsqueeze(2).repeat(1, 1, latent_frames, 1, 1)
        return ((z - mean) / std).float()

    def encode_text(captions: list[str]) -> torch.Tensor:
        length = policy._context_tokens(policy.context_length)
        emb, _ = policy.backend_handle.text(list(captions), length, device, dtype)
        return emb.repeat(2, 1, 1)

    return encode_pixels, encode_text


def train_wan_2_1_dpo(cfg: Any) -> Any:
    from torch.utils.data import DataLoader

    from visionrl_b200.algorithms.dpo import DiffusionDPOConfig
    from visionrl_b200.models.families.wan_2_1.builder import build_wan_2_1_runtime_bundle_from_cfg
    from visionrl_b200.parallel.mesh import ProcessMesh, init_distributed
    from visionrl_b200.trainers.offline_dpo import (
        OfflineDPOTrainer, OfflineDPOTrainerConfig, wan_forward,
    )
    from visionrl_b200.trainers.pickapic import (
        SyntheticLatentPairs, collate_latent_pairs, collate_preference, load_pickapic,
    )

    built = build_configs(cfg)
    algo = built["algorithm"]
    if not isinstance(algo, DiffusionDPOConfig):
        raise TypeError(f"Wan DPO expects algorithm.kind=diffusion_dpo, got {type(algo).__name__}")
    tc = built["trainer"]
    resume = load_training_checkpoint_from_config(cfg)
    prepare_model_config_for_training_resume(cfg, resume, strict=tc.resume_strict)
    native = str(cfg_path(cfg, "distributed.backend", "ray")) == "native"
    rank, world, local = init_distributed(
        timeout_s=float(cfg_path(cfg, "distributed.timeout_s", 1800.0) or 1800.0)) if native else (0, 1, 0)
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    mesh = ProcessMesh.build() if native else ProcessMesh()
    precision = str(require(cfg, "actor.mixed_precision"))
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}.get(precision, torch.float32)
    if device.type == "cpu":
        dtype = torch.float32

    bundle = build_wan_2_1_runtime_bundle_from_cfg(cfg, device, dtype)
    bundle.metadata["family"] = "wan_2_1"
    policy = bundle.policy
    if bool(require(cfg, "actor.gradient_checkpointing")):
        policy.transformer.enable_gradient_checkpointing()
    bundle.scheduler.set_timesteps(1000, device=device)   # index ≈ timestep magnitude

    batch_size = int(require(cfg, "actor.train_batch_size"))
    accum = int(require(cfg, "actor.gradient_accumulation_steps"))
    lr = float(require(cfg, "actor.optim.lr"))
    if bool(require(cfg, "actor.scale_lr")):
        lr *= accum * batch_size * world
    num_frames = int(cfg.sampling.num_frames)
    dpo_cfg = OfflineDPOTrainerConfig(
        beta=algo.beta, sft_weight=algo.sft_weight, lr=lr, scale_lr=False,
        adam_beta1=float(cfg.actor.optim.adam_beta1), adam_beta2=float(cfg.actor.optim.adam_beta2),
        adam_weight_decay=float(cfg.actor.optim.weight_decay),
        adam_epsilon=float(cfg.actor.optim.eps), use_adafactor=bool(require(cfg, "actor.use_adafactor")),
        max_grad_norm=float(cfg.actor.max_norm), gradient_accumulation_steps=accum,
        prediction_type=str(require(cfg, "actor.prediction_type")), num_frames=num_frames,
        mixed_precision=precision, log_every=int(require(cfg, "trainer.log_interval")))
    encode_pixels, encode_text = _build_encoders(policy, num_frames, device, dtype)
    grad_sync = None
    if mesh.world_size > 1:
        from visionrl_b200.parallel.sharded import ShardedGradSync

        grad_sync = ShardedGradSync(mesh, collectives=str(cfg_path(cfg, "distributed.collectives",
                                                                   "fused")))
    ref_model = None if bool(cfg.model.use_lora) else _frozen_copy(policy)
    noise_scheduler = bundle.scheduler
    if dpo_cfg.prediction_type in ("epsilon", "v_prediction"):
        # the flow schedule has no variance-preserving forward process; these targets get one
        from visionrl_b200.models.nn.scheduler import DDPMNoiseScheduler

        noise_scheduler = DDPMNoiseScheduler(prediction_type=dpo_cfg.prediction_type)
        noise_scheduler.set_timesteps(noise_scheduler.num_train_timesteps, device=device)
    trainer = OfflineDPOTrainer(policy, ref_model, wan_forward, noise_scheduler, encode_pixels,
                                encode_text, dpo_cfg, device=device, grad_sync=grad_sync)
    if grad_sync is not None:
        grad_sync.prepare(trainer._optimizer)
    if resume is not None:
        restore_training_checkpoint(resume, trainer=trainer, bundle=bundle, strict=tc.resume_strict)

    resolution = int(require(cfg, "data.resolution")) or int(cfg.sampling.height)
    max_samples = optional_none(cfg, "data.max_train_samples")
    if str(cfg.data.dataset_name) == "synthetic":
        shape = policy.latent_shape(_Request(int(cfg.sampling.height), int(cfg.sampling.width),
                                             num_frames))
        pairs = int(cfg_path(cfg, "data.synthetic.num_pairs", 64))
        dataset = SyntheticLatentPairs(shape, max_samples or pairs,
                                       seed=int(cfg_path(cfg, "data.synthetic.seed", 0)))
        collate = collate_latent_pairs
    else:
        dataset = load_pickapic(split=str(cfg.data.split), cache_dir=str(cfg.data.cache_dir) or None,
                                max_samples=max_samples, resolution=resolution,
                                random_crop=bool(require(cfg, "data.random_crop")),
                                no_hflip=bool(require(cfg, "data.no_hflip")),
                                dataset_name=str(cfg.data.dataset_name))
        collate = collate_preference
    loader_gen = torch.Generator().manual_seed(tc.seed + rank)
    loader = DataLoader(dataset, batch_size=batch_size, shuffle=True, collate_fn=collate,
                        num_workers=int(require(cfg, "data.dataloader_num_workers")),
                        generator=loader_gen, drop_last=True)
    if resume is not None:
        restore_rng_state(resume.rng_state, loader_generator=loader_gen)

    out_dir = Path(tc.output_dir)
    if mesh.is_main:
        out_dir.mkdir(parents=True, exist_ok=True)
        save_resolved_config(cfg, out_dir, resumed=resume is not None)
        prepare_metrics_csv(out_dir / "metrics.csv", DPO_CSV_HEAD, resume=resume is not None)
    max_steps = int(require(cfg, "trainer.max_train_steps"))
    ckpt_every = int(require(cfg, "trainer.checkpointing_steps"))
    step = resume.next_step if resume is not None else 0

    def checkpoint(name: str) -> None:
        if mesh.is_main:
            save_training_checkpoint(
                out_dir / name, trainer=trainer, bundle=bundle, family="wan_2_1",
                progress={"completed_step": step, "next_step": step, "global_step": trainer.global_step},
                rng_state=capture_rng_state(loader_generator=loader_gen))
        else:
            # the same gathers as the writer, in its order (sharded optimiser state, then sharded weights)
            trainer.state_dict()
            join_trainable_state_gathers(bundle)
        mesh.barrier()

    metrics = None
    while step < max_steps:
        for batch in loader:
            metrics = trainer.step(batch)
            step += 1
            if mesh.is_main and step % dpo_cfg.log_every == 0:
                logger.info("step %d | loss=%.5f acc=%.3f model_diff=%.4e ref_diff=%.4e grad_norm=%.4f",
                            step, metrics.loss, metrics.implicit_acc, metrics.model_diff,
                            metrics.ref_diff, metrics.grad_norm)
                with open(out_dir / "metrics.csv", "a") as fh:
                    fh.write(f"{step},{metrics.loss:.6f},{metrics.raw_model_loss:.6f},"
                             f"{metrics.raw_ref_loss:.6f},{metrics.model_diff:.6e},"
                             f"{metrics.ref_diff:.6e},{metrics.implicit_acc:.4f},"
                             f"{metrics.sft_loss:.6f},{metrics.grad_norm:.6f},{lr:.3e}\n")
            if ckpt_every > 0 and step % ckpt_every == 0:
                checkpoint(f"checkpoint-{step}")
            if step >= max_steps:
                break
    checkpoint("checkpoint-final")
    return {"trainer": trainer, "bundle": bundle, "metrics": metrics}


class _Request:
    def __init__(self, height: int, width: int, frames: int) -> None:
        self.height, self.width, self.frame_count = height, width, frames


def _frozen_copy(policy: Any):
    """Frozen reference for full fine-tuning: a deep copy of the transformer."""
    import copy

    class _Ref(torch.nn.Module):
        def __init__(self, transformer):
            super().__init__()
            self.transformer = transformer

    return _Ref(copy.deepcopy(policy.transformer).requires_grad_(False).eval())
