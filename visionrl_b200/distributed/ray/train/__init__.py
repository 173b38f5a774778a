"""Train actors."""
from visionrl_b200.distributed.ray.train.actor import RayTrainActor
from visionrl_b200.distributed.ray.train.group import RayTrainGroup, RayTrainRankSpec

__all__ = ["RayTrainActor", "RayTrainGroup", "RayTrainRankSpec"]
