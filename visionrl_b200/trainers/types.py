"""Trainer configuration and mutable training state (reference: ``vrl/trainers/types.py:8-84``)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(slots=True)
class OptimConfig:
    lr: float = 1e-4
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    weight_decay: float = 1e-4
    eps: float = 1e-8
    use_8bit_adam: bool = False
    allow_tf32: bool = True


@dataclass(slots=True)
class EMAConfig:
    enable: bool = False
    decay: float = 0.9999
    update_interval: int = 1


@dataclass(slots=True)
class DebugConfig:
    first_step: bool = False
    grad_split: bool = False


@dataclass(slots=True)
class TrainerConfig:
    optim: OptimConfig = field(default_factory=OptimConfig)
    ema: EMAConfig = field(default_factory=EMAConfig)
    debug: DebugConfig = field(default_factory=DebugConfig)
    max_norm: float = 1.0
    ppo_epochs: int = 1
    bf16: bool = True
    gradient_checkpointing: bool = True
    n: int = 4
    rollout_batch_size: int = 4
    timestep_fraction: float = 1.0
    total_epochs: int = 10000
    save_freq: int = 50
    log_freq: int = 1
    output_dir: str = "outputs/"
    seed: int = 0
    resume_from: str = ""
    resume_strict: bool = True
    profile: bool = False


@dataclass(slots=True)
class TrainState:
    step: int = 0
    global_step: int = 0
    total_reward: float = 0.0
    total_loss: float = 0.0
