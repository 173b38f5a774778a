"""Worker construction inputs derived from a training config and the family registry
(reference: ``vrl/rollouts/runtime/launch_inputs.py:19-97``): a picklable
``GenerationRuntimeSpec`` for the workers plus a model-free gatherer for the driver."""

from __future__ import annotations

import importlib
from collections.abc import Mapping
from dataclasses import asdict, dataclass
from typing import Any

from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec
from visionrl_b200.engine.gather import ChunkGatherer
from visionrl_b200.rollouts.families import get_rollout_family_entry
from visionrl_b200.rollouts.runtime.config import RolloutBackendConfig, cfg_path


@dataclass(frozen=True, slots=True)
class RolloutRuntimeInputs:
    runtime_spec: GenerationRuntimeSpec
    gatherer: ChunkGatherer


def _import(path: str) -> Any:
    module, attr = path.split(":", 1)
    return getattr(importlib.import_module(module), attr)


def _dtype_name(value: Any) -> str:
    return str(value).removeprefix("torch.")


def build_rollout_runtime_inputs(cfg: Any, family: str, *, weight_dtype: Any,
                                 executor_kwargs: Mapping[str, Any] | None = None,
                                 policy_version: int = 0) -> RolloutRuntimeInputs:
    backend_cfg = RolloutBackendConfig.from_cfg(cfg)
    entry = get_rollout_family_entry(family)
    device = "cuda" if backend_cfg.gpus_per_worker > 0 else "cpu"
    build_spec = _import(entry.runtime_spec_extractor)(cfg, device, _dtype_name(weight_dtype))
    payload = asdict(build_spec)
    payload["device"] = str(payload["device"])
    payload["dtype"] = _dtype_name(payload["dtype"])
    kwargs: dict[str, Any] = {}
    if entry.executor_kwargs.include_sample_batch_size:
        sbs = cfg_path(cfg, "rollout.sample_batch_size", None)
        if sbs is not None:
            kwargs["sample_batch_size"] = int(sbs)
    if entry.executor_kwargs.include_reference_image:
        ref = cfg_path(cfg, "model.reference_image", None)
        if ref:
            kwargs["reference_image"] = str(ref)
    kwargs.update(dict(executor_kwargs or {}))
    return RolloutRuntimeInputs(
        runtime_spec=GenerationRuntimeSpec(
            family=entry.family, task=entry.task, build_spec=payload, executor_kwargs=kwargs,
            policy_version=policy_version, runtime_builder=entry.runtime_builder,
            executor_cls=entry.executor_cls),
        gatherer=_import(entry.gatherer.import_path)(**entry.gatherer.kwargs),
    )


__all__ = ["RolloutRuntimeInputs", "build_rollout_runtime_inputs"]
