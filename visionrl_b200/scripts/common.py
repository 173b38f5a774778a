"""Shared skeleton of the online (GRPO / TokenGRPO) family recipes.

A recipe supplies the family-specific pieces — the runtime bundle, the collector config,
the evaluator, the algorithm — and :func:`run_online_recipe` does what every family does
the same way (reference recipes: ``vrl/scripts/sd3_5/train.py:29-290`` and siblings):
resume handling, reward mix, collector + rollout runtime + weight syncer, trainer
construction, the epoch loop (seeded prompt sampling, ``trainer.step``, log line,
``metrics.csv``, periodic and final checkpoints).

With ``distributed.backend: native`` the same function runs under ``torchrun`` on every
rank: rank ``r`` uses GPU ``LOCAL_RANK``, gradients and optimiser state go through the
sharded runtime, and only rank 0 writes logs, CSV rows and checkpoints.
"""

from __future__ import annotations

import contextlib
import inspect
import logging
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch

from visionrl_b200.config.loader import build_configs, require
from visionrl_b200.rollouts.runtime.config import cfg_path
from visionrl_b200.trainers.checkpointing import (
    LORA_WEIGHTS_NAME, capture_rng_state, join_trainable_state_gathers, load_training_checkpoint_from_config,
    prepare_metrics_csv, prepare_model_config_for_training_resume, restore_rng_state,
    restore_training_checkpoint, sample_prompt_indices, save_resolved_config,
    save_training_checkpoint,
)

logger = logging.getLogger(__name__)

CSV_HEAD = ("epoch,loss,policy_loss,kl_penalty,reward_mean,reward_std,clip_fraction,approx_kl,"
            "advantage_mean,grad_norm,adv_saturation,adv_zero_rate,group_size,trained_prompt_num")


@dataclass
class RecipeParts:
    """What a family recipe hands to :func:`run_online_recipe`."""

    family: str
    bundle: Any
    collector_config: Any
    evaluator: Any
    algorithm: Any
    ref_model: Any = None
    stat_tracker: Any = None
    reference_image: Any = None
    csv_columns: str = CSV_HEAD
    csv_row: Callable[[int, Any], str] | None = None
    first_epoch: int = 0                    # NextStep counts steps from 1
    adapter_module: Any = None              # the module whose adapters a checkpoint exports to
                                            # lora_weights/ (default: the first trainable module)
    extra: dict[str, Any] = field(default_factory=dict)


@dataclass
class RunContext:
    cfg: Any
    built: dict[str, Any]
    trainer_config: Any
    device: torch.device
    weight_dtype: torch.dtype
    mesh: Any
    resume: Any


def setup_run(cfg: Any) -> RunContext:
    """Validate the config, initialise the process group / device and read resume state."""
    from visionrl_b200.parallel.mesh import ProcessMesh, init_distributed

    built = build_configs(cfg)
    tc = built["trainer"]
    if tc.profile:
        os.environ["VRL_PROFILE_COLLECT"] = "1"
    resume = load_training_checkpoint_from_config(cfg)
    prepare_model_config_for_training_resume(cfg, resume, strict=tc.resume_strict)
    native = str(cfg_path(cfg, "distributed.backend", "ray")) == "native"
    rank, world, local = init_distributed(
        timeout_s=float(cfg_path(cfg, "distributed.timeout_s", 1800.0) or 1800.0)) if native else (0, 1, 0)
    if torch.cuda.is_available():
        device = torch.device("cuda", local if native else torch.cuda.current_device())
    else:
        device = torch.device("cpu")
    mesh = ProcessMesh.build(sp=int(cfg_path(cfg, "distributed.mesh.sp", 1) or 1),
                             dp=int(cfg_path(cfg, "distributed.mesh.dp", -1) or -1),
                             fsdp=bool(cfg_path(cfg, "distributed.mesh.fsdp", True)),
                             replicate=int(cfg_path(cfg, "distributed.mesh.replicate", 1) or 1)) \
        if native else ProcessMesh()
    # Sampling noise comes from the default generators: the ranks of one sequence-parallel group
    # must draw identical noise (they hold replicas of the same samples), data-parallel ranks
    # must not, and a rerun with the same seed must reproduce the run.
    torch.manual_seed(int(tc.seed) + 1_000_003 * int(mesh.dp_rank))
    dtype_name = cfg_path(cfg, "model.dtype", None)
    if dtype_name is not None:
        from visionrl_b200.models.families.flow_policy import resolve_dtype

        weight_dtype = resolve_dtype(dtype_name)
    else:
        weight_dtype = torch.bfloat16 if tc.bf16 else torch.float16
    if device.type == "cpu" and weight_dtype == torch.float16:
        weight_dtype = torch.float32
    return RunContext(cfg, built, tc, device, weight_dtype, mesh, resume)


def build_reward(ctx: RunContext):
    from visionrl_b200.rewards.multi import MultiReward

    weights, kwargs = ctx.built["reward"]
    if not weights:
        raise ValueError("At least one reward component must have weight > 0.")
    logger.info("Reward mix: %s", weights)
    return MultiReward.from_dict(weights, device=str(ctx.device), reward_kwargs=kwargs), weights


def _component_means(reward_fn: Any, names: list[str]) -> dict[str, float]:
    means_fn = getattr(reward_fn, "component_means", None)
    got = means_fn() if callable(means_fn) else {}
    last = getattr(reward_fn, "last_components", {}) or {}
    out = {}
    for n in names:
        if n in got:
            out[n] = got[n]
        elif last.get(n):
            out[n] = sum(last[n]) / len(last[n])
        else:
            out[n] = float("nan")
    return out


def default_csv_row(epoch: int, m: Any) -> str:
    return (f"{epoch},{m.loss:.6f},{m.policy_loss:.6f},{m.kl_penalty:.6f},{m.reward_mean:.4f},"
            f"{m.reward_std:.4f},{m.clip_fraction:.4f},{m.approx_kl:.6f},{m.advantage_mean:.6f},"
            f"{m.grad_norm:.6f},{m.adv_saturation:.4f},{m.adv_zero_rate:.4f},{m.group_size:.2f},"
            f"{m.trained_prompt_num}")


def build_online_trainer(ctx: RunContext, parts: RecipeParts, reward_fn: Any):
    """Collector + rollout runtime + weight syncer + (sharded) ``OnlineTrainer`` of a recipe."""
    from visionrl_b200.rollouts.collector import build_rollout_collector
    from visionrl_b200.rollouts.runtime.backend import build_rollout_backend_from_cfg
    from visionrl_b200.rollouts.runtime.launch_inputs import build_rollout_runtime_inputs
    from visionrl_b200.trainers.online import OnlineTrainer
    from visionrl_b200.trainers.weight_sync import build_runtime_weight_syncer

    cfg, tc, bundle, mesh = ctx.cfg, ctx.trainer_config, parts.bundle, ctx.mesh
    policy = bundle.policy
    collector = build_rollout_collector(parts.family, model=policy, reward_fn=reward_fn,
                                        config=parts.collector_config,
                                        reference_image=parts.reference_image)
    executor_kwargs = dict(collector.executor_kwargs)
    inputs = build_rollout_runtime_inputs(cfg, parts.family, weight_dtype=ctx.weight_dtype,
                                          executor_kwargs=executor_kwargs)
    collector.set_runtime(build_rollout_backend_from_cfg(
        cfg, driver_bundle=bundle, runtime_spec=inputs.runtime_spec, gatherer=inputs.gatherer))

    grad_sync = None
    if mesh.world_size > 1:
        from visionrl_b200.parallel.sharded import ShardedGradSync

        collectives = str(cfg_path(cfg, "distributed.collectives", "fused"))
        param_runtime = None
        sharding = str(cfg_path(cfg, "distributed.param_sharding", "full"))
        if mesh.fsdp and sharding == "full":
            from visionrl_b200.parallel.fsdp import shard_model

            # block weights, their gradients and optimiser state live 1/shard-group per rank
            param_runtime = shard_model(
                policy, mesh, ctx.device, collectives=collectives,
                ring=int(cfg_path(cfg, "distributed.gather_ring", 2) or 2),
                rollout_replica=str(cfg_path(cfg, "distributed.weight_sync", "p2p")) != "disabled"
                and bool(cfg_path(cfg, "distributed.rollout_replica", True)))
            if param_runtime is not None:
                policy.param_runtime = param_runtime
                logger.info("sharded %d block weights over %d ranks: %s", len(param_runtime.handles),
                            param_runtime.world, param_runtime.memory_report())
        grad_sync = ShardedGradSync(mesh, shard_optimizer=mesh.fsdp, collectives=collectives,
                                    param_runtime=param_runtime)
    trainer = OnlineTrainer(
        algorithm=parts.algorithm, collector=collector, evaluator=parts.evaluator, model=policy,
        ref_model=parts.ref_model,
        weight_syncer=build_runtime_weight_syncer(
            collector.runtime,
            initial_policy_version=ctx.resume.next_step if ctx.resume is not None else None),
        config=tc, device=ctx.device, stat_tracker=parts.stat_tracker, mesh=mesh,
        grad_sync=grad_sync, liveness=_build_liveness(cfg, mesh))
    if ctx.resume is not None:
        restore_training_checkpoint(ctx.resume, trainer=trainer, bundle=bundle,
                                    strict=tc.resume_strict)
        logger.info("Resuming from %s, start_epoch=%d", ctx.resume.checkpoint_dir,
                    ctx.resume.next_epoch)
    return trainer, collector


def _build_liveness(cfg: Any, mesh: Any):
    """Heartbeats between the ranks of a native multi-rank job (``distributed.heartbeat.*``)."""
    if mesh.world_size <= 1 or not bool(cfg_path(cfg, "distributed.heartbeat.enable", True)):
        return None
    from visionrl_b200.parallel.liveness import build_liveness

    return build_liveness(mesh,
                          interval_s=float(cfg_path(cfg, "distributed.heartbeat.interval_s", 1.0)),
                          deadline_s=float(cfg_path(cfg, "distributed.heartbeat.deadline_s", 60.0)))


def shutdown_distributed(trainer: Any | None = None) -> None:
    """Stop the heartbeat thread and tear the process group down (every recipe's last act)."""
    import torch.distributed as dist

    live = getattr(trainer, "liveness", None)
    if live is not None:
        live.stop()
    if dist.is_available() and dist.is_initialized():
        try:
            dist.barrier()
        except Exception:  # noqa: BLE001 - a peer is already gone; still release our side
            pass
        dist.destroy_process_group()


_CAPTURE: list = [None]


@contextlib.contextmanager
def capture_trainer():
    """While active, a recipe stops after it has built its trainer and hands the pieces back
    (``box["trainer"]``, ``box["examples"]``, ``box["parts"]``, ``box["ctx"]``) instead of running
    its epoch loop.  Benchmarks and smoke tests use this to drive ``trainer.step`` of ANY family's
    recipe themselves, through exactly the objects a training run would use."""
    box: dict[str, Any] = {}
    _CAPTURE[0] = box
    try:
        yield box
    finally:
        _CAPTURE[0] = None


async def run_online_recipe(ctx: RunContext, parts: RecipeParts, reward_fn: Any,
                            reward_names: list[str], *,
                            on_epoch_end: Callable[[int, Any, Any], Any] | None = None,
                            on_checkpoint: Callable[[Path, int, Any, Any], Any] | None = None) -> Any:
    """The epoch loop every online recipe shares.  ``on_epoch_end(epoch, metrics, trainer)`` runs
    after each step on every rank; ``on_checkpoint(directory, completed_epochs, trainer, collector)``
    runs on every rank after each periodic checkpoint (not the final one) and may be a coroutine."""
    from visionrl_b200.trainers.data import load_prompt_manifest

    cfg, tc, bundle, mesh = ctx.cfg, ctx.trainer_config, parts.bundle, ctx.mesh
    trainer, collector = build_online_trainer(ctx, parts, reward_fn)

    manifest = str(require(cfg, "data.manifest"))
    if not manifest.startswith("synthetic:") and not Path(manifest).exists():
        raise FileNotFoundError(f"Manifest not found: {manifest}")
    examples = load_prompt_manifest(manifest)
    if _CAPTURE[0] is not None:
        _CAPTURE[0].update(trainer=trainer, collector=collector, examples=examples, parts=parts,
                           ctx=ctx, reward_fn=reward_fn)
        return _CAPTURE[0]
    start = ctx.resume.next_epoch if ctx.resume is not None else parts.first_epoch
    end = tc.total_epochs + parts.first_epoch
    if start > end:
        raise ValueError("resume checkpoint starts after configured total_epochs: "
                         f"start_epoch={start}, total_epochs={tc.total_epochs}")
    out_dir = Path(tc.output_dir)
    csv_path = out_dir / "metrics.csv"
    if mesh.is_main:
        out_dir.mkdir(parents=True, exist_ok=True)
        save_resolved_config(cfg, out_dir, resumed=ctx.resume is not None)
        header = parts.csv_columns + "".join(f",r_{n}" for n in reward_names) + "\n"
        prepare_metrics_csv(csv_path, header, resume=ctx.resume is not None)
    rng = torch.Generator().manual_seed(tc.seed)
    if ctx.resume is not None:
        restore_rng_state(ctx.resume.rng_state, prompt_generator=rng)
    logger.info("Starting %s training — %d epochs, %d examples, n=%d", parts.family,
                tc.total_epochs, len(examples), tc.n)
    uses_lora = bool(cfg_path(cfg, "model.use_lora", False))
    export = None
    trainable = parts.adapter_module if parts.adapter_module is not None \
        else next(iter(bundle.trainable_modules.values()))
    if uses_lora and hasattr(trainable, "save_pretrained"):
        export = {LORA_WEIGHTS_NAME: trainable}
    row_fn = parts.csv_row or default_csv_row

    def checkpoint(name: str, completed: int) -> None:
        # every rank participates (sharded optimiser state is gathered); rank 0 writes
        state_holder = trainer if mesh.is_main else _StateOnly(trainer)
        target = out_dir / name if mesh.is_main else Path(os.devnull)
        if mesh.is_main:
            save_training_checkpoint(
                target, trainer=state_holder, bundle=bundle, family=parts.family,
                progress={"completed_epoch": completed, "next_epoch": completed,
                          "global_step": trainer.state.global_step},
                rng_state=capture_rng_state(prompt_generator=rng), export_modules=export)
            logger.info("Saved checkpoint to %s", target)
        else:
            # the same gathers, in the writer's order: trainer / optimiser state, then the model
            state_holder.state_dict()
            join_trainable_state_gathers(bundle)
        mesh.barrier()

    metrics = None
    try:
        for epoch in range(start, end):
            picked = sample_prompt_indices(rng, num_examples=len(examples),
                                           rollout_batch_size=tc.rollout_batch_size)
            reset = getattr(reward_fn, "reset_components", None)
            if callable(reset):
                reset()
            step_clock = _StepClock(ctx.device)
            metrics = await trainer.step([examples[i] for i in picked])
            step_ms = step_clock.stop(mesh)
            if mesh.is_main:
                _append_perf(out_dir / "perf.jsonl", epoch, step_ms, trainer, mesh)
            if mesh.is_main and epoch % tc.log_freq == 0:
                comp = _component_means(reward_fn, reward_names)
                logger.info("Epoch %d | loss=%.4f kl=%.4f reward=%.4f+/-%.4f grad_norm=%.4f "
                            "adv_sat=%.3f adv_zero=%.3f | %s", epoch, metrics.loss,
                            metrics.kl_penalty, metrics.reward_mean, metrics.reward_std,
                            metrics.grad_norm, metrics.adv_saturation, metrics.adv_zero_rate,
                            " ".join(f"{n}={comp[n]:.3f}" for n in reward_names))
                with open(csv_path, "a") as fh:
                    fh.write(row_fn(epoch, metrics)
                             + "".join(f",{comp[n]:.4f}" for n in reward_names) + "\n")
            if on_epoch_end is not None:
                on_epoch_end(epoch, metrics, trainer)
            if tc.save_freq > 0 and (epoch + 1 - parts.first_epoch) % tc.save_freq == 0:
                checkpoint(f"checkpoint-{epoch + 1}", epoch + 1)
                if on_checkpoint is not None:
                    pending = on_checkpoint(out_dir / f"checkpoint-{epoch + 1}", epoch + 1, trainer, collector)
                    if inspect.isawaitable(pending):
                        await pending
        if bool(cfg_path(cfg, "trainer.save_final", True)):
            checkpoint("checkpoint-final", end)
            logger.info("Training complete. Final checkpoint: %s", out_dir / "checkpoint-final")
        else:
            logger.info("Training complete (trainer.save_final=false: no final checkpoint written)")
    except BaseException:
        # the step that failed has announced itself to the peers; stop this rank's heartbeats so
        # that whoever restarts the job (the launcher, or scripts/elastic.py in this process)
        # finds no thread writing into a store that is about to go away
        live = getattr(trainer, "liveness", None)
        if live is not None:
            live.stop()
        raise
    shutdown = getattr(collector, "shutdown", None)
    if callable(shutdown):
        await shutdown()
    if bool(cfg_path(cfg, "distributed.destroy_on_exit", True)):
        shutdown_distributed(trainer)
    return {"trainer": trainer, "bundle": bundle, "metrics": metrics}


class _StepClock:
    """Device time of one training step: CUDA events on the current stream (wall clock on CPU),
    the maximum over ranks."""

    def __init__(self, device: torch.device) -> None:
        import time

        self.device = device
        self._t0 = time.perf_counter()
        self._events = None
        if device.type == "cuda":
            self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._events[0].record()

    def stop(self, mesh: Any) -> float:
        import time

        import torch.distributed as dist

        if self._events is not None:
            self._events[1].record()
            self._events[1].synchronize()
            ms = float(self._events[0].elapsed_time(self._events[1]))
        else:
            ms = (time.perf_counter() - self._t0) * 1e3
        if mesh.world_size > 1 and dist.is_available() and dist.is_initialized():
            t = torch.tensor([ms], dtype=torch.float64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms


def _append_perf(path: Path, epoch: int, step_ms: float, trainer: Any, mesh: Any) -> None:
    """One line per step in ``perf.jsonl``: device-timed step, samples per second over the whole
    job, and the kernel-launch count of this rank (kept apart from ``metrics.csv``, whose columns are
    a fixed contract)."""
    import json

    from visionrl_b200.ops import _ext

    dp = max(int(getattr(mesh, "dp", 1)), 1)
    samples = int(getattr(trainer, "last_step_samples", 0)) * dp
    row = {"epoch": epoch, "step_ms": round(step_ms, 3), "samples": samples,
           "samples_per_sec": round(samples / (step_ms / 1e3), 4) if step_ms > 0 else None,
           "n_ranks": int(getattr(mesh, "world_size", 1)), "kernel_launches_total": int(_ext.launch_count)}
    try:
        with open(path, "a") as fh:
            fh.write(json.dumps(row) + "\n")
    except OSError:
        logger.warning("could not append to %s", path, exc_info=True)


class _StateOnly:
    """Non-main ranks still call ``state_dict`` so sharded optimiser state can be gathered."""

    def __init__(self, trainer: Any) -> None:
        self._trainer = trainer

    def state_dict(self) -> dict:
        return self._trainer.state_dict()


def diffusion_collector_kwargs(cfg: Any) -> dict[str, Any]:
    """Fields every diffusion collector config takes from the YAML tree."""
    return dict(
        num_steps=int(cfg.sampling.num_steps), guidance_scale=float(cfg.sampling.guidance_scale),
        height=int(cfg.sampling.height), width=int(cfg.sampling.width),
        noise_level=float(require(cfg, "rollout.noise_level")), cfg=bool(cfg.sampling.cfg),
        sample_batch_size=int(require(cfg, "rollout.sample_batch_size")),
        kl_reward=float(cfg.algorithm.kl_reward), sde_type=str(require(cfg, "rollout.sde.type")),
        sde_window_size=int(cfg.rollout.sde.window_size),
        sde_window_range=tuple(cfg.rollout.sde.window_range),
        same_latent=bool(cfg.rollout.same_latent))


def build_diffusion_parts(ctx: RunContext, family: str, bundle: Any, collector_config: Any,
                          **extra: Any) -> RecipeParts:
    """Evaluator, GRPO algorithm, LoRA reference and stat tracker of a diffusion family."""
    from visionrl_b200.algorithms.grpo import GRPO, GRPOConfig
    from visionrl_b200.algorithms.grpo_token import TokenGRPOConfig
    from visionrl_b200.algorithms.stat_tracking import PerPromptStatTracker
    from visionrl_b200.rollouts.evaluators.diffusion.flow_matching import FlowMatchingEvaluator

    algo_cfg = ctx.built["algorithm"]
    if not isinstance(algo_cfg, GRPOConfig) or isinstance(algo_cfg, TokenGRPOConfig):
        raise TypeError(f"{family} expects algorithm.kind=grpo, got {type(algo_cfg).__name__}")
    cfg = ctx.cfg
    if ctx.trainer_config.gradient_checkpointing:
        enable = getattr(bundle.policy.transformer, "enable_gradient_checkpointing", None)
        if callable(enable):
            enable()
    evaluator = FlowMatchingEvaluator(bundle.scheduler, noise_level=collector_config.noise_level,
                                      sde_type=collector_config.sde_type)
    lora_kl = bool(cfg.model.use_lora) and algo_cfg.init_kl_coef > 0
    tracker = PerPromptStatTracker(global_std=algo_cfg.global_std) \
        if cfg.algorithm.per_prompt_stat_tracking else None
    return RecipeParts(family=family, bundle=bundle, collector_config=collector_config,
                       evaluator=evaluator, algorithm=GRPO(algo_cfg),
                       ref_model=bundle.policy if lora_kl else None, stat_tracker=tracker, **extra)
