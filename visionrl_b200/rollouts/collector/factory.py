"""Builds a :class:`RolloutCollector` from a family name through the family registry
(reference: ``vrl/rollouts/collector/factory.py:26-176``)."""

from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any

from visionrl_b200.engine import RolloutBackend
from visionrl_b200.rollouts.collector.core import RolloutCollector
from visionrl_b200.rollouts.collector.requests import RolloutEngineRequestBuilder
from visionrl_b200.rollouts.collector.rewards import RewardScorer
from visionrl_b200.rollouts.families import FAMILY_REGISTRY, CollectorKind, get_rollout_family_entry
from visionrl_b200.rollouts.packers import (
    ARContinuousRolloutPacker, ARDiscreteRolloutPacker, DiffusionRolloutPacker,
)

# filled by every profiled ``collect`` call; the trainer merges it into its phase report
LAST_COLLECT_PHASES: dict[str, float] = {}


def _import(path: str) -> Any:
    module, attr = path.split(":", 1)
    return getattr(importlib.import_module(module), attr)


@dataclass(frozen=True, slots=True)
class CollectorRegistryEntry:
    family: str
    task: str
    kind: CollectorKind
    config_cls: type
    executor_path: str
    request_prefix: str | None = None
    default_task_type: str | None = None
    error_prefix: str | None = None
    sampling_fields: tuple[str, ...] = ()
    return_artifacts: tuple[str, ...] = ()
    metadata_key: str | None = None

    @property
    def executor_cls(self) -> type:
        return _import(self.executor_path)


COLLECTOR_REGISTRY: dict[str, CollectorRegistryEntry] = {
    family: CollectorRegistryEntry(
        family=e.family, task=e.task, kind=e.collector.kind,
        config_cls=_import(e.collector.config_cls), executor_path=e.executor_cls,
        request_prefix=e.collector.request_prefix, default_task_type=e.collector.default_task_type,
        error_prefix=e.collector.error_prefix, sampling_fields=e.collector.sampling_fields,
        return_artifacts=e.collector.return_artifacts, metadata_key=e.collector.metadata_key,
    )
    for family, e in FAMILY_REGISTRY.items()
}


def _entry(family: str) -> CollectorRegistryEntry:
    if family not in COLLECTOR_REGISTRY:
        raise NotImplementedError(f"no rollout collector registered for family={family!r}; "
                                  f"registered={sorted(COLLECTOR_REGISTRY)}")
    return COLLECTOR_REGISTRY[family]


def collector_config_cls(family: str) -> type:
    return _entry(get_rollout_family_entry(family).family).config_cls


def build_rollout_collector(family: str, *, model: Any | None, reward_fn: Any | None,
                            config: Any | None = None, runtime: RolloutBackend | None = None,
                            reference_image: Any = None) -> RolloutCollector:
    entry = _entry(get_rollout_family_entry(family).family)
    if config is None:
        config = entry.config_cls()
    elif not isinstance(config, entry.config_cls):
        raise TypeError(f"{entry.family} collector requires {entry.config_cls.__name__}, "
                        f"got {type(config).__name__}")
    if entry.request_prefix is None:
        raise ValueError(f"{entry.family} collector registry entry is incomplete")
    builder = RolloutEngineRequestBuilder(
        family=entry.family, task=entry.task, request_prefix=entry.request_prefix, config=config,
        sampling_fields=entry.sampling_fields, return_artifacts=entry.return_artifacts,
        default_task_type=entry.default_task_type, metadata_key=entry.metadata_key,
    )
    if entry.kind == "diffusion":
        packer: Any = DiffusionRolloutPacker(error_prefix=entry.error_prefix or entry.family)
        executor_kwargs: dict[str, Any] = {"sample_batch_size": config.sample_batch_size}
        if reference_image is not None:
            executor_kwargs["reference_image"] = reference_image
        group = 1
    else:
        packer = ARDiscreteRolloutPacker() if entry.kind == "ar_discrete" else ARContinuousRolloutPacker()
        executor_kwargs = {}
        group = int(config.n_samples_per_prompt)
    return RolloutCollector(
        model=model, config=config, family=entry.family, task=entry.task,
        executor_cls=entry.executor_cls, request_builder=builder, packer=packer,
        reward_scorer=RewardScorer(reward_fn), default_group_size=group, runtime=runtime,
        executor_kwargs=executor_kwargs, phase_sink=LAST_COLLECT_PHASES,
    )


__all__ = ["COLLECTOR_REGISTRY", "LAST_COLLECT_PHASES", "CollectorRegistryEntry",
           "build_rollout_collector", "collector_config_cls"]
