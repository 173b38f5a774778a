"""Launches rollout workers and wires executor, weight sync and runtime
(reference: ``vrl/distributed/ray/rollout/launcher.py:23-141``).  A failed policy load
rolls everything back (workers released, placement group removed)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.distributed.ray.placement import create_rollout_placement_group
from visionrl_b200.distributed.ray.rollout.executor import DistributedRolloutExecutor
from visionrl_b200.distributed.ray.rollout.planner import DistributedExecutionPlanner
from visionrl_b200.distributed.ray.rollout.runtime import RayDistributedRuntime
from visionrl_b200.distributed.ray.rollout.types import RayWorkerHandle
from visionrl_b200.distributed.ray.rollout.weight_sync import RayRolloutWeightSync
from visionrl_b200.distributed.ray.rollout.worker import RayRolloutWorker
from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec
from visionrl_b200.engine.gather import require_chunk_gatherer
from visionrl_b200.rollouts.runtime.config import RolloutBackendConfig


class RayRolloutLauncher:
    worker_cls = RayRolloutWorker

    def __init__(self, init_ray: bool = True, ray_init_kwargs: dict[str, Any] | None = None) -> None:
        # kept for the reference's constructor; nothing is initialised, the workers are in-process
        self.init_ray, self.ray_init_kwargs = bool(init_ray), dict(ray_init_kwargs or {})

    def launch(self, config: Any, runtime_spec: Any, gatherer: Any) -> RayDistributedRuntime:
        cfg = RolloutBackendConfig.from_cfg(config)
        spec = GenerationRuntimeSpec.from_value(runtime_spec)
        require_chunk_gatherer(gatherer)
        pg = create_rollout_placement_group(
            cfg.num_workers, gpus_per_worker=cfg.gpus_per_worker,
            cpus_per_worker=cfg.cpus_per_worker, strategy=cfg.placement_strategy)
        transfer = "device" if cfg.gpus_per_worker > 0 else "cpu"
        handles: list[RayWorkerHandle] = []
        try:
            for bundle in pg.bundles:
                worker = self.worker_cls(f"rollout-{bundle.index}", spec, transfer=transfer)
                worker.load_policy()
                handles.append(RayWorkerHandle(
                    worker_id=worker.worker_id, node_id=bundle.node_ip,
                    gpu_ids=() if bundle.gpu_id is None else (bundle.gpu_id,), actor=worker))
        except Exception:
            for h in handles:
                h.actor.release_policy()
            pg.remove()
            raise
        executor = DistributedRolloutExecutor(
            DistributedExecutionPlanner(), handles, gatherer,
            max_inflight_chunks_per_worker=cfg.max_inflight_chunks_per_worker)
        sync = None if cfg.sync_trainable_state == "disabled" else RayRolloutWeightSync(handles)
        return RayDistributedRuntime(executor, handles, sync, pg, spec.policy_version)


def launch_ray_rollout_runtime(config: Any, runtime_spec: Any, gatherer: Any, *, init_ray: bool = True,
                               ray_init_kwargs: dict[str, Any] | None = None) -> RayDistributedRuntime:
    """Function form of :meth:`RayRolloutLauncher.launch`."""
    return RayRolloutLauncher(init_ray, ray_init_kwargs).launch(config, runtime_spec, gatherer)


__all__ = ["RayRolloutLauncher", "launch_ray_rollout_runtime"]
