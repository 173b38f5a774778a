"""Launcher / worker / executor names of the reference's Ray layer
(``vrl/distributed/ray/__init__.py:22-39``), served by in-process workers."""

from visionrl_b200.distributed.ray.placement.group import RayPlacement, create_rollout_placement_group
from visionrl_b200.distributed.ray.rollout.executor import DistributedRolloutExecutor
from visionrl_b200.distributed.ray.rollout.launcher import RayRolloutLauncher, launch_ray_rollout_runtime
from visionrl_b200.distributed.ray.rollout.planner import DeviceAssignment, DistributedExecutionPlanner
from visionrl_b200.distributed.ray.rollout.runtime import RayDistributedRuntime
from visionrl_b200.distributed.ray.rollout.types import RayChunkResult, RayWorkerHandle
from visionrl_b200.distributed.ray.rollout.weight_sync import RayRolloutWeightSync, RolloutWeightSync
from visionrl_b200.distributed.ray.rollout.worker import RayRolloutWorker
from visionrl_b200.distributed.ray.train.actor import RayTrainActor
from visionrl_b200.distributed.ray.train.group import RayTrainGroup, RayTrainRankSpec

__all__ = [
    "DeviceAssignment", "DistributedExecutionPlanner", "DistributedRolloutExecutor",
    "RayChunkResult", "RayDistributedRuntime", "RayPlacement", "RayRolloutLauncher",
    "RayRolloutWeightSync", "RayRolloutWorker", "RayTrainActor", "RayTrainGroup",
    "RayTrainRankSpec", "RayWorkerHandle", "RolloutWeightSync",
    "create_rollout_placement_group", "launch_ray_rollout_runtime",
]
