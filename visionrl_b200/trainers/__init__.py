"""Trainers, checkpointing, EMA, weight synchronisation and prompt data."""

from visionrl_b200.trainers.base import Trainer
from visionrl_b200.trainers.data import DistributedKRepeatSampler, TextPromptDataset
from visionrl_b200.trainers.ema import EMAModuleWrapper
from visionrl_b200.trainers.online import OnlineTrainer
from visionrl_b200.trainers.types import TrainerConfig, TrainState
from visionrl_b200.trainers.weight_sync import (
    InMemoryWeightSyncer, RayRuntimeWeightSyncer, WeightSyncer, build_runtime_weight_syncer,
)

__all__ = [
    "DistributedKRepeatSampler", "EMAModuleWrapper", "InMemoryWeightSyncer", "OnlineTrainer",
    "RayRuntimeWeightSyncer", "TextPromptDataset", "TrainState", "Trainer", "TrainerConfig",
    "WeightSyncer", "build_runtime_weight_syncer",
]
