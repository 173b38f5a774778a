"""Picklable description of how a rollout worker builds its executor.

Only primitives, lists, tuples and string-keyed dicts may appear — tensors,
modules, pipelines and callables are rejected, as are the keys ``executor``,
``policy`` and ``pipeline`` (reference: ``vrl/engine/core/runtime_spec.py:10-195``).
Workers import ``runtime_builder`` and ``executor_cls`` by path.
"""

from __future__ import annotations

import pickle
from collections.abc import Mapping
from dataclasses import dataclass, field, fields
from typing import Any

_LIVE_KEYS = frozenset({"executor", "policy", "pipeline"})
_SCALARS = (str, int, float, bool, type(None))


def _check_plain(value: Any, path: str) -> None:
    if isinstance(value, _SCALARS):
        return
    cls = type(value)
    mod = cls.__module__
    if mod.split(".", 1)[0] == "torch" and cls.__name__ == "Tensor":
        raise TypeError(f"{path} must not contain live torch.Tensor objects")
    if any(c.__module__ == "torch.nn.modules.module" and c.__name__ == "Module" for c in cls.__mro__):
        raise TypeError(f"{path} must not contain live torch.nn.Module objects")
    if mod.startswith("diffusers.") and "Pipeline" in cls.__name__:
        raise TypeError(f"{path} must not contain live diffusers pipeline objects")
    if callable(value):
        raise TypeError(f"{path} must not contain live callable objects")
    if isinstance(value, Mapping):
        for key, inner in value.items():
            if not isinstance(key, str):
                raise TypeError(f"{path} keys must be strings, got {type(key).__name__}")
            _check_plain(inner, f"{path}.{key}")
        return
    if isinstance(value, (list, tuple)):
        for i, inner in enumerate(value):
            _check_plain(inner, f"{path}[{i}]")
        return
    raise TypeError(
        f"{path} must contain only primitive config values, lists, tuples, and dicts; "
        f"got {cls.__name__}"
    )


def _plain_dict(value: Any, path: str) -> dict[str, Any]:
    if value is None:
        return {}
    if not isinstance(value, Mapping):
        raise TypeError(f"{path} must be a dict, got {type(value).__name__}")
    out = dict(value)
    _check_plain(out, path)
    return out


@dataclass(frozen=True, slots=True)
class GenerationRuntimeSpec:
    family: str | None = None
    task: str | None = None
    model_config: dict[str, Any] = field(default_factory=dict)
    executor_kwargs: dict[str, Any] = field(default_factory=dict)
    policy_version: int | None = None
    runtime_builder: str | None = None
    executor_cls: str | None = None
    build_spec: dict[str, Any] | None = None

    def __post_init__(self) -> None:
        set_ = object.__setattr__
        set_(self, "model_config", _plain_dict(self.model_config, "model_config"))
        set_(self, "executor_kwargs", _plain_dict(self.executor_kwargs, "executor_kwargs"))
        if self.build_spec is not None:
            set_(self, "build_spec", _plain_dict(self.build_spec, "build_spec"))
        if self.policy_version is not None:
            set_(self, "policy_version", int(self.policy_version))
        for name in ("runtime_builder", "executor_cls"):
            value = getattr(self, name)
            if value is not None and not isinstance(value, str):
                raise TypeError(f"{name} must be an import path string, got {type(value).__name__}")
        if self.runtime_builder is None or self.executor_cls is None:
            raise ValueError(
                "GenerationRuntimeSpec requires runtime_builder and executor_cls import paths"
            )
        try:
            pickle.dumps(self)
        except Exception as exc:  # noqa: BLE001
            raise TypeError("GenerationRuntimeSpec must be pickle-serializable") from exc

    @classmethod
    def from_value(cls, value: "GenerationRuntimeSpec | Mapping[str, Any]") -> "GenerationRuntimeSpec":
        if isinstance(value, cls):
            return value
        if isinstance(value, Mapping):
            return cls.from_dict(value)
        raise TypeError(
            f"runtime_spec must be a GenerationRuntimeSpec or dict, got {type(value).__name__}"
        )

    @classmethod
    def from_dict(cls, value: Mapping[str, Any]) -> "GenerationRuntimeSpec":
        live = sorted(_LIVE_KEYS.intersection(value))
        if live:
            raise ValueError(
                "GenerationRuntimeSpec cannot include live object keys: "
                + ", ".join(repr(k) for k in live)
                + ". Use runtime_builder and executor_cls import paths instead."
            )
        unknown = sorted(set(value) - {f.name for f in fields(cls)})
        if unknown:
            raise ValueError(
                "unsupported GenerationRuntimeSpec keys: " + ", ".join(repr(k) for k in unknown)
                + ". Put model payload under model_config or executor_kwargs."
            )
        return cls(**dict(value))

    def to_dict(self) -> dict[str, Any]:
        return {
            "family": self.family, "task": self.task, "model_config": dict(self.model_config),
            "executor_kwargs": dict(self.executor_kwargs), "policy_version": self.policy_version,
            "runtime_builder": self.runtime_builder, "executor_cls": self.executor_cls,
            "build_spec": None if self.build_spec is None else dict(self.build_spec),
        }

    def build_spec_payload(self) -> dict[str, Any]:
        return dict(self.build_spec if self.build_spec is not None else self.model_config)


__all__ = ["GenerationRuntimeSpec"]
