"""Generic collector: build request → runtime.generate → score rewards → pack
(reference: ``vrl/rollouts/collector/core.py:20-163``).  With
``VRL_PROFILE_COLLECT=1`` the two sub-phases are timed into ``phase_sink``."""

from __future__ import annotations

import os
import time
from collections.abc import Mapping
from typing import Any

from visionrl_b200.engine import OutputBatch, RolloutBackend
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.collector.requests import RolloutRequestBuilder, RolloutRequestPlan
from visionrl_b200.rollouts.collector.rewards import RewardScorer
from visionrl_b200.rollouts.packers.base import RolloutPackContext, RolloutPacker


def _now_synced() -> float:
    import torch

    if torch.cuda.is_available():
        torch.cuda.synchronize()
    return time.perf_counter()


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

    async def shutdown(self) -> None:
        stop = getattr(self._runtime, "shutdown", None)
        if stop is not None:
            await stop()
        self._runtime = None

    async def release_runtime_memory(self) -> None:
        release = getattr(self._runtime, "release_memory", None)
        if release is not None:
            await release()

    async def collect(self, prompts: list[str], **kwargs: Any) -> RolloutBatch:
        group_size = int(kwargs.get("group_size", self.default_group_size))
        plan = self.request_builder.build(prompts, group_size, dict(kwargs))
        profile = os.environ.get("VRL_PROFILE_COLLECT") == "1"
        phases: dict[str, float] = {}
        t0 = _now_synced() if profile else 0.0
        output = await self.runtime.generate(plan.request)
        if output.error:
            raise RuntimeError(f"{self.family}/{self.task} generation failed "
                               f"(request_id={plan.request.request_id}): {output.error}")
        if profile:
            t1 = _now_synced()
            phases["collect.engine_generate"] = t1 - t0
            t0 = t1
        batch = await self._to_rollout_batch(output, plan)
        if profile:
            phases["collect.reward_score"] = _now_synced() - t0
            if self.phase_sink is not None:
                self.phase_sink.clear()
                self.phase_sink.update(phases)
        return batch

    async def _to_rollout_batch(self, output: OutputBatch, plan: RolloutRequestPlan) -> RolloutBatch:
        ctx = RolloutPackContext(
            metadata=dict(plan.pack_metadata), device=getattr(self.model, "device", None),
            kl_reward=float(getattr(self.config, "kl_reward", 0.0)),
            rescale_to_unit=bool(getattr(self.config, "rescale_to_unit", False)),
        )
        outputs = self.packer.reward_outputs(output, ctx)
        device = ctx.device if ctx.device is not None else getattr(outputs, "device", "cpu")
        rewards = await self.reward_scorer.score(outputs, self.packer.reward_prompts(output, ctx),
                                                 plan.reward_metadata, device)
        return await self.packer.pack(output, rewards, ctx)


__all__ = ["RolloutCollector"]
