"""Worker placement."""
from visionrl_b200.distributed.ray.placement.group import (
    PlacementBundle, RayPlacement, RolloutPlacementGroup, create_rollout_placement_group,
)
from visionrl_b200.distributed.ray.placement.network import sort_node_gpu_key

__all__ = ["PlacementBundle", "RayPlacement", "RolloutPlacementGroup", "create_rollout_placement_group",
           "sort_node_gpu_key"]
