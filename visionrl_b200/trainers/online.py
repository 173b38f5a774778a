"""Online RL trainer: collect → advantages → per-group, per-timestep replay → update.

One ``step``:

1. the current weights are pushed to the rollout runtime before the very first
   collect (and again after every update);
2. plain-string prompts are collected in ONE request of ``n`` samples each, rich
   ``PromptExample`` items one request each (their reward metadata is per prompt);
   the result is split into one batch per prompt group;
3. advantages come from the per-prompt stat tracker (then zero-advantage samples are
   dropped) or from the algorithm's group normalisation; in a multi-rank job the
   rewards / group ids of all ranks are gathered first so groups split across ranks
   are normalised together;
4. for every PPO epoch, every group batch and every trained timestep the evaluator
   replays the policy, the algorithm forms the loss (divided by the number of
   groups), and gradients accumulate; then one clipped optimiser step and one EMA
   update;
5. metrics are accumulated on the device and read back once per step.

Behavioural reference: ``vrl/trainers/online.py:233-851``.
"""

from __future__ import annotations

import contextlib
import json
import logging
import os
import time
from typing import Any

import torch
from torch import nn

from visionrl_b200.algorithms.base import Algorithm
from visionrl_b200.algorithms.types import TrainStepMetrics
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.trainers.base import Trainer, raise_on_kernel_timeout
from visionrl_b200.trainers.ema import EMAModuleWrapper
from visionrl_b200.trainers.types import TrainerConfig, TrainState
from visionrl_b200.trainers.weight_sync import WeightSyncer

logger = logging.getLogger(__name__)


def _nvtx_wanted() -> bool:
    return os.environ.get("VRL_NVTX", "0") == "1" and torch.cuda.is_available()


class PhaseTimer:
    """Named accumulating timer; synchronises the device around each phase when CUDA is up.

    With ``VRL_NVTX=1`` every phase is also an NVTX range (``vrl/<phase>``), whether or not the
    timer itself is enabled, so a timeline profiler shows the step's structure without the
    synchronisation that exact phase times need."""

    def __init__(self, enabled: bool = False, sync: bool = True) -> None:
        self.enabled = enabled
        self.sync = bool(sync) and torch.cuda.is_available()
        self.times: dict[str, float] = {}
        self.events: list[tuple[str, float, float]] = []
        self._nvtx = _nvtx_wanted()

    @contextlib.contextmanager
    def time(self, name: str):
        if self._nvtx:
            torch.cuda.nvtx.range_push(f"vrl/{name}")
        try:
            if not self.enabled:
                yield
                return
            if self.sync:
                torch.cuda.synchronize()
            t0, w0 = time.perf_counter(), time.time()
            try:
                yield
            finally:
                if self.sync:
                    torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                self.times[name] = self.times.get(name, 0.0) + dt
                self.events.append((name, w0, w0 + dt))
        finally:
            if self._nvtx:
                torch.cuda.nvtx.range_pop()


def create_optimizer(params: list, config: TrainerConfig):
    o = config.optim
    if o.use_8bit_adam:
        try:
            import bitsandbytes as bnb

            return bnb.optim.AdamW8bit(params, lr=o.lr, betas=(o.adam_beta1, o.adam_beta2),
                                       weight_decay=o.weight_decay, eps=o.eps)
        except ImportError:
            logger.warning("use_8bit_adam=true but bitsandbytes is missing; using fused AdamW")
    from visionrl_b200.ops.optim import FusedAdamW

    return FusedAdamW(params, lr=o.lr, betas=(o.adam_beta1, o.adam_beta2),
                      weight_decay=o.weight_decay, eps=o.eps)


def apply_sample_mask(batch: RolloutBatch, mask: torch.Tensor) -> RolloutBatch:
    n = batch.rewards.shape[0]
    extras = {k: (v[mask] if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] == n else v)
              for k, v in batch.extras.items()}
    prompts = None
    if batch.prompts is not None:
        prompts = [p for p, keep in zip(batch.prompts, mask.detach().cpu().tolist(), strict=True)
                   if keep]
    return RolloutBatch(
        observations=batch.observations[mask], actions=batch.actions[mask],
        rewards=batch.rewards[mask], dones=batch.dones[mask], group_ids=batch.group_ids[mask],
        extras=extras, context=batch.context,
        videos=batch.videos[mask] if batch.videos is not None else None, prompts=prompts)


def split_batch_by_group(batch: RolloutBatch) -> list[RolloutBatch]:
    order: list[int] = []
    for gid in batch.group_ids.detach().cpu().tolist():
        if int(gid) not in order:
            order.append(int(gid))
    if len(order) <= 1:
        return [batch]
    return [apply_sample_mask(batch, batch.group_ids == gid) for gid in order]


def remap_group_ids_(batch: RolloutBatch, global_indices: list[int]) -> None:
    """Collector-local prompt indices → trainer-global prompt indices."""
    if not global_indices:
        return
    table = torch.as_tensor(global_indices, dtype=batch.group_ids.dtype, device=batch.group_ids.device)
    batch.group_ids = table[batch.group_ids]


def _move_tree(value: Any, device: torch.device) -> Any:
    if isinstance(value, torch.Tensor):
        return value if value.device == device else value.to(device)
    if isinstance(value, dict):
        return {k: _move_tree(v, device) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_move_tree(v, device) for v in value)
    return value


def move_training_batch(batch: RolloutBatch, device: torch.device) -> RolloutBatch:
    """Replay tensors to the trainer device (a no-op when rollout ran there); frames stay put."""
    return RolloutBatch(
        observations=_move_tree(batch.observations, device), actions=_move_tree(batch.actions, device),
        rewards=_move_tree(batch.rewards, device), dones=_move_tree(batch.dones, device),
        group_ids=_move_tree(batch.group_ids, device), extras=_move_tree(batch.extras, device),
        context=_move_tree(batch.context, device), videos=batch.videos, prompts=batch.prompts)


def _autocast(cfg: TrainerConfig, device: torch.device, model: nn.Module):
    """bf16 autocast only for fp32 weights on CUDA; bf16-weight models need none."""
    if not cfg.bf16 or device.type != "cuda":
        return contextlib.nullcontext()
    first = next((p for p in model.parameters()), None)
    if first is not None and first.dtype != torch.float32:
        return contextlib.nullcontext()
    return torch.amp.autocast("cuda", dtype=torch.bfloat16)


class OnlineTrainer(Trainer):
    _grad_split_already_fired = False

    def __init__(self, algorithm: Algorithm, collector: Any, evaluator: Any, model: nn.Module,
                 ref_model: nn.Module | None = None, weight_syncer: WeightSyncer | None = None,
                 config: TrainerConfig | None = None, prompts: list[str] | None = None,
                 device: torch.device | str = "cuda", accelerator: Any | None = None,
                 stat_tracker: Any | None = None, mesh: Any | None = None,
                 grad_sync: Any | None = None, liveness: Any | None = None) -> None:
        self.algorithm, self.collector, self.evaluator = algorithm, collector, evaluator
        self.model, self.ref_model, self.weight_syncer = model, ref_model, weight_syncer
        self.config = config or TrainerConfig()
        self.prompts = prompts or []
        self.device = torch.device(device) if isinstance(device, str) else device
        self.state = TrainState()
        self.accelerator = accelerator
        self.stat_tracker = stat_tracker
        self.mesh = mesh
        self.grad_sync = grad_sync
        # host-side heartbeats of a multi-rank job (visionrl_b200.parallel.liveness.RankLiveness)
        self.liveness = liveness
        self._optimizer: torch.optim.Optimizer | None = None
        self._ema: EMAModuleWrapper | None = None
        self._rollout_weights_initialized = False
        self.last_step_samples = 0
        self.last_d2h_bytes = 0
        if self.config.optim.allow_tf32:
            torch.backends.cuda.matmul.allow_tf32 = True

    # -- lazy pieces -----------------------------------------------------------------
    def _trainable(self) -> list[nn.Parameter]:
        return [p for p in self.model.parameters() if p.requires_grad]

    def _ensure_optimizer(self) -> torch.optim.Optimizer:
        if self._optimizer is None:
            self._optimizer = create_optimizer(self._trainable(), self.config)
            prepare = getattr(self.grad_sync, "prepare", None)
            if callable(prepare):
                prepare(self._optimizer)
        return self._optimizer

    def _ensure_ema(self) -> EMAModuleWrapper | None:
        if not self.config.ema.enable:
            return None
        if self._ema is None:
            self._ema = EMAModuleWrapper(self._trainable(), decay=self.config.ema.decay,
                                         update_step_interval=self.config.ema.update_interval,
                                         device=self.device)
        return self._ema

    async def _ensure_rollout_weights_initialized(self) -> None:
        if self._rollout_weights_initialized or self.weight_syncer is None:
            return
        await self.weight_syncer.push(self._sync_payload())
        self._rollout_weights_initialized = True

    async def push_rollout_weights(self) -> None:
        """Send the current trainable state to the rollout workers now (a no-op without a syncer)."""
        if self.weight_syncer is not None:
            await self.weight_syncer.push(self._sync_payload())
            self._rollout_weights_initialized = True

    # -- optimisation helpers ------------------------------------------------------------
    def _sync_payload(self) -> dict:
        """What a weight push carries: the trainable set when the policy can name it (adapters
        only under LoRA), otherwise the whole ``state_dict()``."""
        export = getattr(self.model, "trainable_state_dict", None)
        return export() if callable(export) else self.model.state_dict()

    def _backward(self, loss: Any) -> None:
        if self.accelerator is not None:
            self.accelerator.backward(loss)
        else:
            from visionrl_b200.ops.linear import accumulate_weight_grads_in_place

            # weight gradients are summed into the existing .grad buffers by the GEMM itself
            with accumulate_weight_grads_in_place():
                loss.backward()

    def _clip_and_step(self, optimizer: Any) -> Any:
        """Clip, step, zero.  Returns the pre-clip gradient norm (tensor or float)."""
        cfg = self.config
        if self.grad_sync is not None:
            norm = self.grad_sync.reduce_clip_step(optimizer, cfg.max_norm)
            return norm
        fused_norm = getattr(optimizer, "grad_norm", None)
        if self.accelerator is not None:
            norm: Any = 0.0
            if self.accelerator.sync_gradients and cfg.max_norm > 0:
                norm = self.accelerator.clip_grad_norm_(self.model.parameters(), cfg.max_norm)
            optimizer.step()
        elif callable(fused_norm):
            norm = fused_norm()
            coef = None
            if cfg.max_norm > 0:
                coef = (cfg.max_norm / (norm + 1e-6)).clamp(max=1.0)
            optimizer.step(clip_coef=coef)
        else:
            if cfg.max_norm > 0:
                norm = nn.utils.clip_grad_norm_(self.model.parameters(), cfg.max_norm)
            else:
                grads = [p.grad.detach().float().pow(2).sum() for p in self.model.parameters()
                         if p.grad is not None]
                norm = torch.stack(grads).sum().sqrt() if grads else torch.zeros(())
            optimizer.step()
        optimizer.zero_grad()
        return norm

    def _clear_algorithm_diagnostics(self) -> None:
        for attr in ("_last_policy_loss_tensor", "_last_kl_term_tensor"):
            if hasattr(self.algorithm, attr):
                setattr(self.algorithm, attr, None)

    # -- phases of a step -----------------------------------------------------------------
    async def _collect(self, cfg: TrainerConfig) -> list[RolloutBatch]:
        from visionrl_b200.trainers.data import PromptExample

        batches: list[RolloutBatch] = []
        plain: list[str] = []
        plain_idx: list[int] = []

        async def flush() -> None:
            if not plain:
                return
            b = await self.collector.collect(list(plain), group_size=cfg.n)
            remap_group_ids_(b, plain_idx)
            batches.extend(split_batch_by_group(b))
            plain.clear()
            plain_idx.clear()

        items = list(enumerate(self.prompts))
        mesh = self.mesh
        runtime = getattr(self.collector, "_runtime", None)
        if mesh is not None and getattr(mesh, "dp", 1) > 1 and hasattr(runtime, "split_chunks"):
            # whole prompt groups per data-parallel rank when there are enough prompts;
            # otherwise the runtime splits the chunks of each group across ranks
            shard_prompts = len(items) >= mesh.dp and len(items) % mesh.dp == 0
            runtime.split_chunks = not shard_prompts
            if shard_prompts:
                items = items[mesh.dp_rank::mesh.dp]
        for idx, item in items:
            if isinstance(item, PromptExample):
                await flush()
                b = await self.collector.collect(
                    [item.prompt], group_size=cfg.n, target_text=item.target_text,
                    references=item.references, task_type=item.task_type,
                    request_overrides=item.request_overrides, sample_metadata=item.metadata)
                b.group_ids[:] = idx
                batches.extend(split_batch_by_group(b))
            else:
                plain.append(str(item))
                plain_idx.append(idx)
        await flush()
        return batches

    def _gather_rewards(self, rewards: torch.Tensor, group_ids: torch.Tensor):
        """Rewards / group ids of every data-parallel rank (this rank's slice location too)."""
        mesh = self.mesh
        if mesh is None or getattr(mesh, "dp", 1) <= 1:
            return rewards, group_ids, 0
        group = getattr(mesh, "dp_group", None)
        r_parts = mesh.all_gather_varlen(rewards.float().contiguous(), group)
        g_parts = mesh.all_gather_varlen(group_ids.to(torch.float32).contiguous(), group)
        start = sum(p.numel() for p in r_parts[: mesh.dp_rank])
        return torch.cat(r_parts), torch.cat(g_parts).to(group_ids.dtype), start

    def _advantages(self, batches: list[RolloutBatch]):
        local_rewards = torch.cat([b.rewards for b in batches])
        local_groups = torch.cat([b.group_ids for b in batches])
        rewards, groups, start = self._gather_rewards(local_rewards, local_groups)
        group_size, trained = 0.0, 0
        clip_max = getattr(self.algorithm.config, "adv_clip_max", None)
        if self.stat_tracker is not None:
            prompts = [p for b in batches for p in (b.prompts or [])]
            if rewards.numel() != local_rewards.numel():
                prompts = [f"group:{int(g)}" for g in groups.tolist()]
            adv_np = self.stat_tracker.update(prompts, rewards)
            group_size, trained = self.stat_tracker.get_stats()
            self.stat_tracker.clear()
            adv = torch.as_tensor(adv_np, dtype=torch.float32, device=rewards.device)
            if clip_max is not None:
                adv = adv.clamp(-clip_max, clip_max)
        else:
            adv = self.algorithm.compute_advantages_from_tensors(rewards, groups)
        total = max(adv.numel(), 1)
        absadv = adv.detach().abs()
        stats = torch.stack([
            (absadv < 1e-6).sum().float() / total,
            ((absadv >= clip_max - 1e-6).sum().float() / total) if clip_max is not None
            else absadv.new_zeros(()),
            rewards.float().mean(),
            rewards.float().std() if rewards.numel() > 1 else rewards.new_zeros(()).float(),
            adv.float().mean(),
        ])
        local_adv = adv[start:start + local_rewards.numel()]
        return local_adv, stats, group_size, trained

    def _filter(self, batches, adv_split):
        if self.stat_tracker is None:
            return list(batches), list(adv_split)
        kept_b, kept_a = [], []
        for b, a in zip(batches, adv_split, strict=True):
            mask = a.detach().abs() != 0
            if not bool(mask.any()):
                a = a + 1e-6
                mask = a.detach().abs() != 0
            if not bool(mask.all()):
                b, a = apply_sample_mask(b, mask), a[mask]
            if b.rewards.shape[0] > 0:
                kept_b.append(b)
                kept_a.append(a)
        return kept_b, kept_a

    def _train_indices(self, num_timesteps: int) -> list[int]:
        count = max(1, int(num_timesteps * self.config.timestep_fraction))
        if count >= num_timesteps:
            return list(range(num_timesteps))
        return [int(i * num_timesteps / count) for i in range(count)]

    def _debug_first_step(self, batch: RolloutBatch, ctx) -> None:
        from visionrl_b200.rollouts.evaluators.types import SignalRequest

        old = batch.extras["log_probs"]
        with ctx, torch.no_grad():
            sig = self.evaluator.evaluate(self.model, batch, 0, ref_model=self.ref_model,
                                          signal_request=SignalRequest())
        old0 = old[:, 0] if old.ndim > 1 else old
        diff = (sig.log_prob - old0).abs()
        logger.info("DEBUG first-step log-prob diff: mean=%.6f max=%.6f | old_lp[0]=%.6f "
                    "fresh_lp[0]=%.6f", diff.mean().item(), diff.max().item(),
                    old0.reshape(-1)[0].item(), sig.log_prob.reshape(-1)[0].item())
        self.last_first_step_diff = float(diff.max().item())

    def _grad_split(self, j: int) -> None:
        p_t = getattr(self.algorithm, "_last_policy_loss_tensor", None)
        k_t = getattr(self.algorithm, "_last_kl_term_tensor", None)
        params = self._trainable()

        def norm_of(term):
            if term is None or not term.requires_grad:
                return float("nan")
            grads = torch.autograd.grad(term, params, retain_graph=True, allow_unused=True)
            return float(sum((g.detach().float() ** 2).sum() for g in grads if g is not None) ** 0.5)

        pn, kn = norm_of(p_t), norm_of(k_t)
        ratio = pn / kn if kn and kn > 0 else float("inf")
        logger.info("[GRAD-SPLIT RESULT] step=%d j=%d ||grad(policy)||=%.4e ||grad(beta*kl)||=%.4e "
                    "policy/kl_ratio=%.3f", self.state.step, j, pn, kn, ratio)

    def _write_phase_events(self, timer: PhaseTimer, phase_times: dict[str, float]) -> None:
        cfg = self.config
        total = sum(v for k, v in phase_times.items() if not k.startswith("collect.")) or 1.0
        parts = " | ".join(f"{k}={v:.3f}s ({100 * v / total:.1f}%)" for k, v in phase_times.items())
        logger.info("phase_times[step=%d] total=%.3fs | %s", self.state.step, total, parts)
        try:
            os.makedirs(cfg.output_dir, exist_ok=True)
            with open(os.path.join(cfg.output_dir, "phase_events.jsonl"), "a") as fh:
                for name, start, end in timer.events:
                    fh.write(json.dumps({"step": self.state.step, "phase": name, "start": start,
                                         "end": end}) + "\n")
            timer.events.clear()
        except OSError:
            logger.warning("could not write phase_events.jsonl", exc_info=True)

    # -- the step ------------------------------------------------------------------------------
    async def step(self, prompts: list[str] | None = None) -> TrainStepMetrics:
        """One policy step.  In a multi-rank job the peers' liveness is checked first (a rank that
        failed or fell silent ends this rank with ``RankFailure`` before anything is launched),
        and an exception raised here is announced to the peers before it propagates."""
        live = self.liveness
        if live is not None:
            live.check()
            live.beat(self.state.step)
        try:
            if os.environ.get("VRL_FAULT_INJECT"):
                from visionrl_b200.parallel.liveness import maybe_inject_fault

                maybe_inject_fault(live.rank if live is not None else 0, self.state.step)
            return await self._step(prompts)
        except BaseException as exc:
            if live is not None:
                live.announce_failure(f"{type(exc).__name__}: {exc}")
            raise

    async def _step(self, prompts: list[str] | None = None) -> TrainStepMetrics:
        from visionrl_b200.rollouts.evaluators.types import SignalRequest

        if prompts is not None:
            self.prompts = prompts
        cfg = self.config
        optimizer = self._ensure_optimizer()
        ema = self._ensure_ema()
        timer = PhaseTimer(enabled=cfg.profile)
        await self._ensure_rollout_weights_initialized()

        runtime = getattr(self.collector, "_runtime", None)
        offload = self.device.type == "cuda" and bool(
            getattr(runtime, "requires_driver_model_offload", False))
        if offload:
            with timer.time("offload_driver_model"):
                self.model.to("cpu")
                torch.cuda.empty_cache()
        with timer.time("collect"):
            batches = await self._collect(cfg)
        with timer.time("release_rollout"):
            release = getattr(self.collector, "release_runtime_memory", None)
            if callable(release):
                await release()
        if offload:
            with timer.time("restore_driver_model"):
                self.model.to(self.device)

        with timer.time("advantage"):
            adv_local, adv_stats, group_size, trained_prompts = self._advantages(batches)
            sizes = [b.rewards.shape[0] for b in batches]
            kept, kept_adv = self._filter(batches, list(torch.split(adv_local, sizes)))
        self.last_step_samples = sum(sizes)

        if not kept:
            logger.info("step %d: all batches filtered (zero advantages); skipping backward",
                        self.state.step)
            self.state.step += 1
            s = adv_stats.tolist()
            return TrainStepMetrics(reward_mean=s[2], reward_std=s[3], advantage_mean=s[4],
                                    adv_zero_rate=s[0], adv_saturation=s[1],
                                    phase_times=dict(timer.times))

        self.model.train()
        ctx = _autocast(cfg, self.device, self.model)
        kept = [move_training_batch(b, self.device) for b in kept]
        kept_adv = [a.to(self.device) for a in kept_adv]
        train_indices = self._train_indices(kept[0].observations.shape[1])
        num_accum = len(kept)
        if cfg.debug.first_step and self.state.step == 0:
            self._debug_first_step(kept[0], ctx)
            runtime_check = getattr(getattr(self.model, "param_runtime", None), "verify_replicas", None)
            if runtime_check is not None:
                runtime_check()             # every rank rolled out with the same weights

        need_ref = self.algorithm.config.init_kl_coef > 0
        request = SignalRequest(need_ref=need_ref, need_kl_intermediates=need_ref)
        device_metrics = hasattr(self.algorithm, "sync_metrics")
        previous_sync = getattr(self.algorithm, "sync_metrics", True)
        if device_metrics:
            self.algorithm.sync_metrics = False
        metric_rows: list[Any] = []
        host_rows: list[TrainStepMetrics] = []
        grad_norms: list[Any] = []
        try:
            for _epoch in range(cfg.ppo_epochs):
                for b, adv_b in zip(kept, kept_adv, strict=True):
                    old_lp = b.extras["log_probs"]
                    for j in train_indices:
                        with timer.time("evaluate"), ctx:
                            signals = self.evaluator.evaluate(self.model, b, j,
                                                              ref_model=self.ref_model,
                                                              signal_request=request)
                            old_j = old_lp[:, j] if old_lp.ndim > 1 else old_lp
                            loss, metrics = self.algorithm.compute_signal_loss(signals, adv_b, old_j)
                            loss = loss / num_accum
                        if cfg.debug.grad_split and not OnlineTrainer._grad_split_already_fired:
                            OnlineTrainer._grad_split_already_fired = True
                            try:
                                self._grad_split(j)
                            except Exception as exc:  # noqa: BLE001
                                logger.warning("debug_grad_split failed: %s", exc)
                        with timer.time("backward"):
                            self._backward(loss)
                        row = getattr(self.algorithm, "last_metric_tensor", None) if device_metrics else None
                        if row is not None:
                            metric_rows.append(row)
                        else:
                            host_rows.append(metrics)
                        self._clear_algorithm_diagnostics()
                with timer.time("optim_step"):
                    grad_norms.append(self._clip_and_step(optimizer))
                if ema is not None:
                    ema.step(self._trainable(), self.state.global_step)
                self.state.global_step += 1
        finally:
            if device_metrics:
                self.algorithm.sync_metrics = previous_sync

        # single device→host read of everything this step produced
        if metric_rows:
            means = torch.stack(metric_rows).float().mean(dim=0)
        elif host_rows:
            means = torch.tensor([[m.loss, m.policy_loss, m.kl_penalty, m.clip_fraction, m.approx_kl]
                                  for m in host_rows]).mean(dim=0)
        else:
            means = torch.zeros(5)
        gn = torch.stack([torch.as_tensor(g, dtype=torch.float32).reshape(()).to(means.device)
                          for g in grad_norms]).mean() if grad_norms else means.new_zeros(())
        packed = torch.cat([means.to(adv_stats.device), adv_stats.float(),
                            gn.reshape(1).to(adv_stats.device)]).tolist()
        loss_v, pol_v, kl_v, clip_v, akl_v, zero_v, sat_v, r_mean, r_std, a_mean, gn_v = packed
        self.last_d2h_bytes = 4 * len(packed)
        self._check_kernel_status()

        phase_times = dict(timer.times)
        if cfg.profile:
            try:
                from visionrl_b200.rollouts.collector import LAST_COLLECT_PHASES

                phase_times.update(LAST_COLLECT_PHASES)
            except Exception:  # noqa: BLE001
                pass
            if phase_times:
                self._write_phase_events(timer, phase_times)

        out = TrainStepMetrics(
            loss=loss_v, policy_loss=pol_v, kl_penalty=kl_v, reward_mean=r_mean, reward_std=r_std,
            advantage_mean=a_mean, clip_fraction=clip_v, approx_kl=akl_v, grad_norm=gn_v,
            adv_saturation=sat_v, adv_zero_rate=zero_v, lr=float(cfg.optim.lr),
            group_size=group_size, trained_prompt_num=trained_prompts, phase_times=phase_times)
        self.state.step += 1
        self.state.total_reward += out.reward_mean
        self.state.total_loss += out.loss
        if self.weight_syncer is not None:
            await self.weight_syncer.push(self._sync_payload())
        return out

    def _check_kernel_status(self) -> None:
        """Bounded device-side waits report here instead of hanging; raise if one gave up."""
        self.last_d2h_bytes += raise_on_kernel_timeout(self.device, self.grad_sync,
                                                       f"training step {self.state.step}")

    # -- state -------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        d: dict[str, Any] = {"step": self.state.step, "global_step": self.state.global_step,
                             "total_reward": self.state.total_reward,
                             "total_loss": self.state.total_loss}
        if self._optimizer is not None:
            d["optimizer"] = self._optimizer.state_dict()
        if self._ema is not None:
            d["ema"] = self._ema.state_dict()
        return d

    def load_state_dict(self, state: dict, *, strict: bool = True) -> None:
        if not isinstance(state, dict):
            raise TypeError("OnlineTrainer.load_state_dict expects a dict")
        self.state.step = int(state.get("step", 0))
        self.state.global_step = int(state.get("global_step", 0))
        self.state.total_reward = float(state.get("total_reward", 0.0))
        self.state.total_loss = float(state.get("total_loss", 0.0))
        if "optimizer" in state:
            try:
                self._ensure_optimizer().load_state_dict(state["optimizer"])
            except Exception:
                if strict:
                    raise
                logger.warning("Skipping incompatible optimizer state during non-strict load")
        if "ema" in state:
            if not self.config.ema.enable:
                if strict:
                    raise ValueError("checkpoint contains EMA state but trainer.ema.enable=false")
                logger.warning("Skipping EMA state because trainer.ema.enable=false")
            else:
                try:
                    self._ensure_ema().load_state_dict(state["ema"])
                except Exception:
                    if strict:
                        raise
                    logger.warning("Skipping incompatible EMA state during non-strict load")
        # the rollout side must receive the restored weights before the next collect
        self._rollout_weights_initialized = False


__all__ = ["OnlineTrainer", "PhaseTimer", "apply_sample_mask", "create_optimizer",
           "move_training_batch", "remap_group_ids_", "split_batch_by_group"]
