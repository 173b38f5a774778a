"""Native rollout runtime: every rank of the job generates its share of the chunks.

All ranks receive the same ``GenerationRequest``.  The prompt-major micro-batch plan
is cut round-robin over the data-parallel ranks (ranks of one sequence-parallel
group run the same chunks together); each rank runs its chunks on its own GPU and
returns an ``OutputBatch`` holding only its samples — the latent trajectories stay
in that rank's HBM and are trained on there.  Only rewards and group ids (a few
floats per sample) ever cross ranks, when the trainer normalises advantages.

The executor is either built from the picklable runtime spec or wraps the live
policy of the colocated trainer (``driver_policy``), in which case rollout and
training share one set of weights on the GPU and no weight transfer is needed.
"""

from __future__ import annotations

import dataclasses
from typing import Any

from visionrl_b200.distributed.ray.module_loading import import_from_path
from visionrl_b200.distributed.ray.rollout.planner import request_chunks
from visionrl_b200.distributed.ray.rollout.worker import build_executor_from_spec
from visionrl_b200.engine.core.runtime import stamp_policy_version
from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec
from visionrl_b200.engine.core.types import GenerationRequest, OutputBatch
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.gather import gather_pipeline_chunks, require_chunk_gatherer, require_chunked_executor
from visionrl_b200.engine.microbatching import BisectingRunner
from visionrl_b200.parallel.mesh import ProcessMesh
from visionrl_b200.rollouts.runtime.config import RolloutBackendConfig


class NativeRolloutRuntime:
    def __init__(self, executor: Any, gatherer: Any, mesh: ProcessMesh, *,
                 policy_version: int | None = None, shares_trainer_weights: bool = False,
                 sync_enabled: bool = True) -> None:
        self.executor = require_chunked_executor(executor)
        self.gatherer = require_chunk_gatherer(gatherer)
        self.mesh = mesh
        self.id_factory = GenerationIdFactory()
        self.current_policy_version = policy_version
        self.shares_trainer_weights = shares_trainer_weights
        self.weight_sync = object() if sync_enabled else None
        self.requires_driver_model_offload = False
        self.last_local_chunks = 0
        self.last_bisections = 0
        # False: the caller already handed this rank only its own prompts
        self.split_chunks = True

    def local_chunks(self, request: GenerationRequest):
        """This rank's share of the request's chunk list (every rank derives the same list)."""
        plan = request_chunks(request)
        if not self.split_chunks or self.mesh.dp <= 1:
            return list(plan.micro_batches)
        return list(plan.for_rank(self.mesh.dp_rank, self.mesh.dp))

    async def generate(self, request: GenerationRequest) -> OutputBatch:
        request = stamp_policy_version(request, self.current_policy_version)
        chunks = self.local_chunks(request)
        self.last_local_chunks = len(chunks)
        if not chunks:
            raise RuntimeError(
                f"rank {self.mesh.rank} received no rollout chunks: the request has fewer "
                f"micro-batches than data-parallel ranks ({self.mesh.dp})")
        runner = BisectingRunner(lambda c: self.executor.forward_chunk(request, c))
        results = runner.run(chunks)
        self.last_bisections = runner.bisections
        # the runner knows which samples every result holds, also after a chunk was bisected
        spec_of = {(s.prompt_index, s.sample_index): s
                   for s in self.id_factory.build_sample_specs(request)}
        specs = [spec_of[(c.prompt_index, j)] for c in runner.executed
                 for j in range(c.sample_start, c.sample_end)]
        return gather_pipeline_chunks(self.gatherer, request, specs, results)

    async def update_weights(self, state_ref: Any, policy_version: int) -> None:
        """Bring the rollout copy to ``policy_version``.

        With shared weights the trainer already wrote the parameters the rollout reads;
        otherwise ``state_ref`` is a name → tensor mapping (device tensors are copied
        device-to-device) or a callable performing the device-side broadcast.
        """
        if not self.shares_trainer_weights and state_ref is not None:
            if callable(state_ref):
                state_ref(self.executor.model)
            else:
                self.executor.model.load_trainable_state(state_ref)
        self.current_policy_version = int(policy_version)

    async def release_memory(self) -> None:
        return None

    async def shutdown(self) -> None:
        return None


class NativeRolloutLauncher:
    def launch(self, config: Any, runtime_spec: Any, gatherer: Any, *,
               driver_policy: Any | None = None, mesh: ProcessMesh | None = None) -> NativeRolloutRuntime:
        cfg = RolloutBackendConfig.from_cfg(config)
        spec = GenerationRuntimeSpec.from_value(runtime_spec)
        mesh = mesh or ProcessMesh.current() or ProcessMesh.build()
        if driver_policy is not None and cfg.allow_driver_gpu_overlap:
            executor = import_from_path(str(spec.executor_cls))(
                driver_policy, **dict(spec.executor_kwargs))
            shared = True
        else:
            executor = build_executor_from_spec(spec)
            shared = False
        return NativeRolloutRuntime(
            executor, gatherer, mesh, policy_version=spec.policy_version,
            shares_trainer_weights=shared, sync_enabled=cfg.sync_trainable_state != "disabled")


__all__ = ["NativeRolloutLauncher", "NativeRolloutRuntime"]
