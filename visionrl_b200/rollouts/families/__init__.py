"""Rollout family registry."""

from visionrl_b200.rollouts.families.specs import (
    DIFFUSION_COMMON_SAMPLING_FIELDS, DIFFUSION_RETURN_ARTIFACTS, DIFFUSION_VIDEO_SAMPLING_FIELDS,
    FAMILY_REGISTRY, CollectorKind, CollectorMetadata, ExecutorKwargsMetadata, GathererMetadata,
    RolloutFamilyEntry, get_rollout_family_entry, normalize_rollout_family,
    registered_rollout_families,
)

__all__ = [
    "DIFFUSION_COMMON_SAMPLING_FIELDS", "DIFFUSION_RETURN_ARTIFACTS",
    "DIFFUSION_VIDEO_SAMPLING_FIELDS", "FAMILY_REGISTRY", "CollectorKind", "CollectorMetadata",
    "ExecutorKwargsMetadata", "GathererMetadata", "RolloutFamilyEntry",
    "get_rollout_family_entry", "normalize_rollout_family", "registered_rollout_families",
]
