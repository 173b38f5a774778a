"""Rollout workers, planner, executor and runtime."""
from visionrl_b200.distributed.ray.rollout.executor import DistributedRolloutExecutor
from visionrl_b200.distributed.ray.rollout.launcher import RayRolloutLauncher, launch_ray_rollout_runtime
from visionrl_b200.distributed.ray.rollout.planner import DeviceAssignment, DistributedExecutionPlanner
from visionrl_b200.distributed.ray.rollout.runtime import RayDistributedRuntime
from visionrl_b200.distributed.ray.rollout.types import RayChunkResult, RayWorkerHandle
from visionrl_b200.distributed.ray.rollout.weight_sync import RayRolloutWeightSync, RolloutWeightSync
from visionrl_b200.distributed.ray.rollout.worker import RayRolloutWorker

__all__ = [
    "DeviceAssignment", "DistributedExecutionPlanner", "DistributedRolloutExecutor", "RayChunkResult",
    "RayDistributedRuntime", "RayRolloutLauncher", "RayRolloutWeightSync", "RayRolloutWorker", "RayWorkerHandle",
    "RolloutWeightSync", "launch_ray_rollout_runtime",
]
