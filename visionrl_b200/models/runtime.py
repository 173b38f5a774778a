"""Builder input / output types (reference: ``vrl/models/runtime.py:15-62``).

``RuntimeBundle.trainable_modules`` is the checkpoint contract: generic trainer
checkpointing saves and restores exactly these ``name → module`` entries.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class RuntimeBuildSpec:
    model_name_or_path: str
    device: Any
    dtype: Any
    backend_preference: tuple[str, ...] = ("native",)
    task_variant: str | None = None
    mixed_precision: str | None = None
    use_lora: bool = False
    lora_path: str | None = None
    lora_config: dict[str, Any] | None = None
    offload_config: dict[str, Any] | None = None
    scheduler_config: dict[str, Any] | None = None
    native_backend_config: dict[str, Any] | None = None
    diffusers_backend_config: dict[str, Any] | None = None
    extra: dict[str, Any] = field(default_factory=dict)


@dataclass
class RuntimeBundle:
    policy: Any
    trainable_modules: dict[str, Any]
    scheduler: Any
    backend_kind: str
    backend_handle: Any
    ref_modules: dict[str, Any] | None = None
    runtime_caps: dict[str, Any] = field(default_factory=dict)
    metadata: dict[str, Any] = field(default_factory=dict)


__all__ = ["RuntimeBuildSpec", "RuntimeBundle"]
