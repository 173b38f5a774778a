"""Worker placement."""
from visionrl_b200.distributed.ray.placement.group import (
    PlacementBundle, RolloutPlacementGroup, create_rollout_placement_group,
)

__all__ = ["PlacementBundle", "RolloutPlacementGroup", "create_rollout_placement_group"]
