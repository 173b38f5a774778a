"""Builds the engine request of one ``collect`` call from the collector config
(reference: ``vrl/rollouts/collector/requests.py:12-136``).  Only the sampling fields
declared for the family are copied; tuples become lists; a seed and per-call
``request_overrides`` are applied last."""

from __future__ import annotations

import uuid
from dataclasses import dataclass, field
from typing import Any, Protocol

from visionrl_b200.engine import GenerationRequest


@dataclass(slots=True)
class RolloutRequestPlan:
    request: GenerationRequest
    reward_metadata: dict[str, Any] = field(default_factory=dict)
    pack_metadata: dict[str, Any] = field(default_factory=dict)


class RolloutRequestBuilder(Protocol):
    def build(self, prompts: list[str], group_size: int, kwargs: dict[str, Any]) -> RolloutRequestPlan: ...


class RolloutEngineRequestBuilder:
    def __init__(self, *, family: str, task: str, request_prefix: str, config: Any,
                 sampling_fields: tuple[str, ...], return_artifacts: tuple[str, ...],
                 default_task_type: str | None = None, metadata_key: str | None = None) -> None:
        if not sampling_fields:
            raise ValueError(f"{family} request builder requires sampling_fields")
        if not return_artifacts:
            raise ValueError(f"{family} request builder requires return_artifacts")
        self.family, self.task, self.request_prefix = family, task, request_prefix
        self.config = config
        self.sampling_fields, self.return_artifacts = sampling_fields, return_artifacts
        self.default_task_type, self.metadata_key = default_task_type, metadata_key

    def _sampling(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for name in self.sampling_fields:
            if not hasattr(self.config, name):
                raise ValueError(f"{type(self.config).__name__} is missing sampling field {name!r}")
            value = getattr(self.config, name)
            out[name] = list(value) if isinstance(value, tuple) else value
        return out

    def _metadata(self, kwargs: dict[str, Any]) -> dict[str, Any]:
        meta: dict[str, Any] = dict(kwargs.get("sample_metadata") or {})
        for key in ("target_text", "references"):
            if kwargs.get(key):
                meta[key] = kwargs[key]
        if self.default_task_type is not None:
            meta["task_type"] = kwargs.get("task_type", self.default_task_type)
            if kwargs.get("reference_image") is not None:
                meta["reference_image"] = kwargs["reference_image"]
        return meta

    def build(self, prompts: list[str], group_size: int, kwargs: dict[str, Any]) -> RolloutRequestPlan:
        sampling = self._sampling()
        if kwargs.get("seed") is not None:
            sampling["seed"] = kwargs["seed"]
        sampling.update(dict(kwargs.get("request_overrides", {}) or {}))
        meta = self._metadata(kwargs)
        request = GenerationRequest(
            request_id=f"{self.request_prefix}-{uuid.uuid4()}", family=self.family, task=self.task,
            prompts=prompts, samples_per_prompt=group_size, sampling=sampling,
            return_artifacts=set(self.return_artifacts),
            metadata={self.metadata_key: dict(meta)} if self.metadata_key else dict(meta),
            policy_version=kwargs.get("policy_version"),
        )
        return RolloutRequestPlan(request=request, reward_metadata=meta, pack_metadata=meta)


__all__ = ["RolloutEngineRequestBuilder", "RolloutRequestBuilder", "RolloutRequestPlan"]
