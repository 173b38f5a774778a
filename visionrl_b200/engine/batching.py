"""Fusion of identically configured requests into one executor call.

Requests are mergeable only if family, task, group size, the full sampling dict,
artifact set and policy version agree.  The merged prompt-major output is cut
back per request: every tensor (or nested container of tensors) whose leading
dimension equals the merged sample count is sliced
(reference: ``vrl/engine/batching.py:30-275``).
"""

from __future__ import annotations

import dataclasses
from typing import Any

from visionrl_b200.engine.core.types import GenerationRequest, GenerationSampleSpec, OutputBatch


def _check_mergeable(requests: list[GenerationRequest]) -> None:
    head = requests[0]
    for other in requests[1:]:
        if (other.family, other.task) != (head.family, head.task):
            raise ValueError("Cannot merge requests from different family/task")
        if other.samples_per_prompt != head.samples_per_prompt:
            raise ValueError("Cannot merge requests with different sample counts")
        if other.sampling != head.sampling:
            raise ValueError("Cannot merge requests with different sampling config")
        if other.return_artifacts != head.return_artifacts:
            raise ValueError("Cannot merge requests with different artifact modes")
        if other.policy_version != head.policy_version:
            raise ValueError("Cannot merge requests with different policy versions")


def slice_leading(value: Any, offset: int, count: int, total: int) -> Any:
    """Slice ``value`` along dim 0 wherever that dim has length ``total``."""
    if value is None:
        return None
    shape = getattr(value, "shape", None)
    if shape is not None and hasattr(value, "__getitem__"):
        return value[offset:offset + count] if len(shape) > 0 and shape[0] == total else value
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        changes = {f.name: slice_leading(getattr(value, f.name), offset, count, total)
                   for f in dataclasses.fields(value)}
        return dataclasses.replace(value, **changes)
    if isinstance(value, dict):
        return {k: slice_leading(v, offset, count, total) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        if len(value) == total:
            return type(value)(value[offset:offset + count])
        return type(value)(slice_leading(v, offset, count, total) for v in value)
    return value


def forward_batch_by_merging_prompts(
    executor: Any,
    requests: list[GenerationRequest],
    sample_specs_by_request: dict[str, list[GenerationSampleSpec]],
) -> dict[str, OutputBatch]:
    if not requests:
        return {}
    if len(requests) == 1:
        only = requests[0]
        return {only.request_id: executor.forward(only, sample_specs_by_request[only.request_id])}
    _check_mergeable(requests)
    head = requests[0]
    prompts = [p for r in requests for p in r.prompts]
    specs = [s for r in requests for s in sample_specs_by_request[r.request_id]]
    merged = GenerationRequest(
        request_id=f"batch:{head.request_id}", family=head.family, task=head.task,
        prompts=prompts, samples_per_prompt=head.samples_per_prompt, sampling=dict(head.sampling),
        return_artifacts=set(head.return_artifacts),
        metadata={"batched_request_ids": [r.request_id for r in requests]},
        priority=min(r.priority for r in requests), policy_version=head.policy_version,
    )
    out = executor.forward(merged, specs)
    total = len(specs)
    results: dict[str, OutputBatch] = {}
    offset = 0
    for r in requests:
        own = sample_specs_by_request[r.request_id]
        n = len(own)
        cut = lambda v, o=offset, c=n: slice_leading(v, o, c, total)  # noqa: E731
        results[r.request_id] = OutputBatch(
            request_id=r.request_id, family=r.family, task=r.task, prompts=list(r.prompts),
            sample_specs=own, output=cut(out.output),
            trajectory_timesteps=cut(out.trajectory_timesteps),
            trajectory_latents=cut(out.trajectory_latents),
            rollout_trajectory_data=cut(out.rollout_trajectory_data),
            trajectory_decoded=cut(out.trajectory_decoded), extra=cut(out.extra),
            metrics=out.metrics, peak_memory_mb=out.peak_memory_mb, error=out.error,
        )
        offset += n
    return results


__all__ = ["forward_batch_by_merging_prompts", "slice_leading"]
