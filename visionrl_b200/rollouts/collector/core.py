"""The collector of every family: request → rollout backend → rewards → ``RolloutBatch``.

What differs between families is injected — the request builder (which sampling fields a family
declares), the packer (how an ``OutputBatch`` becomes observations / actions / extras) and the
reward scorer — so this class holds only the sequence and the plumbing around it:

1. build one ``GenerationRequest`` for the prompts (``group_size`` samples each);
2. hand it to the rollout backend.  In a multi-rank job every rank makes the same call and gets
   back the samples IT generated; nothing is gathered across ranks here;
3. score the decoded outputs and pack.  Outputs, rewards and the packed batch stay on the
   device of the policy.

With ``VRL_PROFILE_COLLECT=1`` the time of step 2 and of step 3 (each fenced by a device
synchronise) is written into ``phase_sink`` for the trainer's phase report.  Behavioural
reference: ``vrl/rollouts/collector/core.py:20-163``.
"""

from __future__ import annotations

import contextlib
import os
import time
from collections.abc import Mapping
from typing import Any

from visionrl_b200.engine import OutputBatch, RolloutBackend
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.collector.requests import RolloutRequestBuilder, RolloutRequestPlan
from visionrl_b200.rollouts.collector.rewards import RewardScorer
from visionrl_b200.rollouts.packers.base import RolloutPackContext, RolloutPacker


class _PhaseClock:
    """Device-fenced wall-clock timing of named phases; inert unless enabled."""

    def __init__(self, enabled: bool) -> None:
        self.enabled = enabled
        self.seconds: dict[str, float] = {}

    @staticmethod
    def _fence() -> float:
        import torch

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return time.perf_counter()

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        start = self._fence()
        try:
            yield
        finally:
            self.seconds[name] = self.seconds.get(name, 0.0) + self._fence() - start


class RolloutCollector:
    def __init__(self, *, model: Any | None, config: Any, family: str, task: str,
                 executor_cls: type, request_builder: RolloutRequestBuilder, packer: RolloutPacker,
                 reward_scorer: RewardScorer, default_group_size: int = 1,
                 runtime: RolloutBackend | None = None,
                 executor_kwargs: Mapping[str, Any] | None = None,
                 phase_sink: dict[str, float] | None = None) -> None:
        self.model, self.config, self.family, self.task = model, config, family, task
        self.executor_cls = executor_cls
        self.request_builder, self.packer, self.reward_scorer = request_builder, packer, reward_scorer
        self.default_group_size = max(1, int(default_group_size))
        self._runtime = runtime
        self.executor_kwargs = dict(executor_kwargs or {})
        self.phase_sink = phase_sink

    # -- the backend this collector talks to -------------------------------------------------
    def set_runtime(self, runtime: RolloutBackend) -> None:
        if not callable(getattr(runtime, "generate", None)):
            raise TypeError("rollout runtime must implement async generate(request) -> OutputBatch")
        self._runtime = runtime

    @property
    def runtime(self) -> RolloutBackend:
        if self._runtime is None:
            raise RuntimeError("RolloutCollector runtime is not initialized; "
                               "call set_runtime(...) before collect(...)")
        return self._runtime

    async def _call_runtime(self, method: str) -> None:
        fn = getattr(self._runtime, method, None)
        if fn is not None:
            await fn()

    async def release_runtime_memory(self) -> None:
        await self._call_runtime("release_memory")

    async def shutdown(self) -> None:
        await self._call_runtime("shutdown")
        self._runtime = None

    # -- collecting -------------------------------------------------------------------------------
    def _pack_context(self, plan: RolloutRequestPlan) -> RolloutPackContext:
        cfg = self.config
        return RolloutPackContext(metadata=dict(plan.pack_metadata),
                                  device=getattr(self.model, "device", None),
                                  kl_reward=float(getattr(cfg, "kl_reward", 0.0)),
                                  rescale_to_unit=bool(getattr(cfg, "rescale_to_unit", False)))

    async def _score_and_pack(self, output: OutputBatch, plan: RolloutRequestPlan) -> RolloutBatch:
        ctx = self._pack_context(plan)
        scored = self.packer.reward_outputs(output, ctx)
        device = ctx.device if ctx.device is not None else getattr(scored, "device", "cpu")
        rewards = await self.reward_scorer.score(scored, self.packer.reward_prompts(output, ctx),
                                                 plan.reward_metadata, device)
        return await self.packer.pack(output, rewards, ctx)

    async def collect(self, prompts: list[str], **kwargs: Any) -> RolloutBatch:
        group_size = int(kwargs.get("group_size", self.default_group_size))
        plan = self.request_builder.build(prompts, group_size, dict(kwargs))
        clock = _PhaseClock(os.environ.get("VRL_PROFILE_COLLECT") == "1")
        with clock.phase("collect.engine_generate"):
            output = await self.runtime.generate(plan.request)
            if output.error:
                raise RuntimeError(f"{self.family}/{self.task} generation failed "
                                   f"(request_id={plan.request.request_id}): {output.error}")
        with clock.phase("collect.reward_score"):
            batch = await self._score_and_pack(output, plan)
        if clock.enabled and self.phase_sink is not None:
            self.phase_sink.clear()
            self.phase_sink.update(clock.seconds)
        return batch


__all__ = ["RolloutCollector"]
