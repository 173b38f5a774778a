"""Collectors: request building, reward scoring and the generic collect loop."""

from visionrl_b200.rollouts.collector.base import Collector
from visionrl_b200.rollouts.collector.configs import (
    CosmosPredict2CollectorConfig, JanusProCollectorConfig, NextStep1CollectorConfig,
    SD3_5CollectorConfig, Wan_2_1CollectorConfig,
)
from visionrl_b200.rollouts.collector.core import RolloutCollector
from visionrl_b200.rollouts.collector.factory import (
    COLLECTOR_REGISTRY, LAST_COLLECT_PHASES, CollectorRegistryEntry, build_rollout_collector,
    collector_config_cls,
)

__all__ = [
    "COLLECTOR_REGISTRY", "LAST_COLLECT_PHASES", "Collector", "CollectorRegistryEntry",
    "CosmosPredict2CollectorConfig", "JanusProCollectorConfig", "NextStep1CollectorConfig",
    "RolloutCollector", "SD3_5CollectorConfig", "Wan_2_1CollectorConfig",
    "build_rollout_collector", "collector_config_cls",
]
