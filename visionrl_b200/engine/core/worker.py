"""Local generation worker: expands requests into sample specs, fuses
same-configuration requests and turns executor exceptions into
``OutputBatch.error`` (reference: ``vrl/engine/core/worker.py:19-217``).

Sample ids are ``"<request>:prompt:<i>:sample:<j>"``; a request-level seed gives
sample ``k`` (prompt-major flat index) the seed ``base + k``.
"""

from __future__ import annotations

import logging
from typing import Any

from visionrl_b200.engine.core.registry import FamilyPipelineRegistry
from visionrl_b200.engine.core.types import (
    GenerationMetrics, GenerationRequest, GenerationSampleSpec, OutputBatch,
)

logger = logging.getLogger(__name__)


class GenerationIdFactory:
    def build_sample_specs(self, request: GenerationRequest) -> list[GenerationSampleSpec]:
        base = request.sampling.get("seed")
        base = None if base is None else int(base)
        specs: list[GenerationSampleSpec] = []
        for p_idx, prompt in enumerate(request.prompts):
            prompt_id = f"{request.request_id}:prompt:{p_idx}"
            for s_idx in range(request.samples_per_prompt):
                flat = len(specs)
                sample_id = f"{prompt_id}:sample:{s_idx}"
                meta = {**request.metadata, "request_id": request.request_id, "prompt_index": p_idx,
                        "sample_index": s_idx, "flat_sample_index": flat,
                        "policy_version": request.policy_version}
                specs.append(GenerationSampleSpec(
                    prompt_index=p_idx, sample_index=s_idx, prompt=prompt, prompt_id=prompt_id,
                    group_id=prompt_id, sample_id=sample_id, trajectory_id=sample_id,
                    seed=None if base is None else base + flat, metadata=meta,
                ))
        return specs


def _freeze(value: Any) -> Any:
    if isinstance(value, dict):
        return tuple((k, _freeze(v)) for k, v in sorted(value.items()))
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(v) for v in value)
    if isinstance(value, set):
        return tuple(sorted(_freeze(v) for v in value))
    try:
        hash(value)
    except TypeError:
        return repr(value)
    return value


def _fusion_key(request: GenerationRequest) -> tuple[Any, ...]:
    s = request.sampling
    # seeded requests and SDE-window requests are never merged with others
    if "seed" in s or int(s.get("sde_window_size", 0)) > 0:
        return (request.request_id,)
    return (request.family, request.task, request.samples_per_prompt, request.policy_version,
            tuple(sorted(request.return_artifacts)), _freeze(s))


def _error_output(request: GenerationRequest, specs: list[Any], error: str) -> OutputBatch:
    return OutputBatch(
        request_id=request.request_id, family=request.family, task=request.task,
        prompts=list(request.prompts), sample_specs=specs, output=None,
        metrics=GenerationMetrics(num_prompts=len(request.prompts), num_samples=len(specs)),
        error=error,
    )


class GenerationWorker:
    def __init__(self, registry: FamilyPipelineRegistry, *,
                 id_factory: GenerationIdFactory | None = None, device: Any | None = None):
        self.registry = registry
        self.id_factory = id_factory or GenerationIdFactory()
        self.device = device

    def execute(self, requests: list[GenerationRequest]) -> dict[str, OutputBatch]:
        groups: dict[Any, list[GenerationRequest]] = {}
        for request in requests:
            groups.setdefault(_fusion_key(request), []).append(request)
        outputs: dict[str, OutputBatch] = {}
        for group in groups.values():
            if len(group) == 1:
                outputs[group[0].request_id] = self._execute_one(group[0])
            else:
                outputs.update(self._execute_group(group))
        return outputs

    def _execute_one(self, request: GenerationRequest) -> OutputBatch:
        specs = self.id_factory.build_sample_specs(request)
        try:
            executor = self.registry.resolve(request.family, request.task)
            out = executor.forward(request, specs)
            if out.request_id != request.request_id:
                raise ValueError(
                    f"Executor returned request_id={out.request_id!r} for "
                    f"request_id={request.request_id!r}"
                )
            return out
        except Exception as exc:  # noqa: BLE001 - reported through OutputBatch.error
            logger.exception("Generation request %s failed", request.request_id)
            return _error_output(request, specs, str(exc))

    def _execute_group(self, requests: list[GenerationRequest]) -> dict[str, OutputBatch]:
        specs = {r.request_id: self.id_factory.build_sample_specs(r) for r in requests}
        try:
            executor = self.registry.resolve(requests[0].family, requests[0].task)
            fused = getattr(executor, "forward_batch", None)
            if fused is None:
                return {r.request_id: self._execute_one(r) for r in requests}
            outs = fused(requests, specs)
            return {
                r.request_id: outs.get(r.request_id) or _error_output(
                    r, specs[r.request_id],
                    "Batched executor did not return an output for this request")
                for r in requests
            }
        except Exception as exc:  # noqa: BLE001
            logger.exception("Generation request batch failed: %s", [r.request_id for r in requests])
            return {r.request_id: _error_output(r, specs[r.request_id], str(exc)) for r in requests}
