"""YAML configuration: loader, validators and typed config builders."""

from visionrl_b200.config.cli import parse_and_load
from visionrl_b200.config.loader import (
    CONFIGS_ROOT,
    build_algorithm_config,
    build_configs,
    build_reward_config,
    build_trainer_config,
    load_config,
    optional_none,
    require,
    validate_reward_config,
    validate_training_config,
)
from visionrl_b200.config.node import DictConfig, ListConfig, OmegaConf

__all__ = [
    "CONFIGS_ROOT", "DictConfig", "ListConfig", "OmegaConf", "build_algorithm_config",
    "build_configs", "build_reward_config", "build_trainer_config", "load_config",
    "optional_none", "parse_and_load", "require", "validate_reward_config", "validate_training_config",
]
