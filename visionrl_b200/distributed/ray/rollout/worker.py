"""Rollout worker: builds its executor from a picklable runtime spec, runs chunks,
applies weight updates and reports stale policy versions as chunk errors
(reference: ``vrl/distributed/ray/rollout/worker.py:19-213``).

``transfer="cpu"`` moves chunk payloads to host memory (what an object store
needs); ``transfer="device"`` keeps them where they were produced.
"""

from __future__ import annotations

import dataclasses
import gc
from collections.abc import Mapping
from typing import Any

from visionrl_b200.distributed.ray.dependencies import current_gpu_ids, current_node_ip
from visionrl_b200.distributed.ray.module_loading import import_from_path
from visionrl_b200.distributed.ray.rollout.types import RayChunkResult
from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.gather import require_chunked_executor
from visionrl_b200.engine.microbatching import MicroBatchPlan


def to_cpu(value: Any) -> Any:
    if hasattr(value, "detach") and hasattr(value, "cpu"):
        return value.detach().cpu()
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return type(value)(**{f.name: to_cpu(getattr(value, f.name))
                              for f in dataclasses.fields(value)})
    if isinstance(value, dict):
        return {k: to_cpu(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(to_cpu(v) for v in value)
    return value


def build_executor_from_spec(runtime_spec: GenerationRuntimeSpec) -> Any:
    if runtime_spec.runtime_builder is None or runtime_spec.executor_cls is None:
        raise ValueError(
            "GenerationRuntimeSpec requires runtime_builder and executor_cls import paths")
    import torch

    from visionrl_b200.models.families.flow_policy import resolve_dtype
    from visionrl_b200.models.runtime import RuntimeBuildSpec

    payload = dict(runtime_spec.build_spec_payload())
    if isinstance(payload.get("device"), str):
        payload["device"] = torch.device(payload["device"])
    if isinstance(payload.get("dtype"), str):
        try:
            payload["dtype"] = resolve_dtype(payload["dtype"])
        except ValueError as exc:
            raise ValueError(
                f"unsupported torch dtype string in runtime_spec: {payload['dtype']!r}") from exc
    if "backend_preference" in payload:
        payload["backend_preference"] = tuple(payload["backend_preference"])
    bundle = import_from_path(str(runtime_spec.runtime_builder))(RuntimeBuildSpec(**payload))
    executor = import_from_path(str(runtime_spec.executor_cls))(
        bundle.policy, **dict(runtime_spec.executor_kwargs))
    return require_chunked_executor(executor)


class RayRolloutWorker:
    def __init__(self, worker_id: str, runtime_spec: GenerationRuntimeSpec | Mapping[str, Any],
                 transfer: str = "cpu") -> None:
        self.worker_id = worker_id
        self.runtime_spec = GenerationRuntimeSpec.from_value(runtime_spec)
        if self.runtime_spec.family is None:
            raise ValueError("GenerationRuntimeSpec.family is required")
        self.family = self.runtime_spec.family
        self.executor: Any | None = None
        self.transfer = transfer
        self._policy_version: int | None = self.runtime_spec.policy_version

    def load_policy(self) -> None:
        if self.executor is None:
            self.executor = build_executor_from_spec(self.runtime_spec)

    def release_policy(self) -> None:
        self.executor = None
        gc.collect()
        try:
            import torch

            if torch.cuda.is_available():
                torch.cuda.empty_cache()
                torch.cuda.ipc_collect()
        except Exception:  # noqa: BLE001
            pass

    def update_weights(self, state_ref: Any, policy_version: int) -> None:
        self.load_policy()
        if state_ref is not None:
            policy = getattr(self.executor, "model", None)
            if policy is None:
                raise RuntimeError(f"{type(self.executor).__name__} must expose model for weight sync")
            apply_state = getattr(policy, "load_trainable_state", None)
            if not callable(apply_state):
                raise RuntimeError(f"{type(policy).__name__} must implement load_trainable_state()")
            apply_state(state_ref)
        self._policy_version = int(policy_version)

    def current_policy_version(self) -> int | None:
        return self._policy_version

    def worker_metadata(self) -> dict[str, Any]:
        try:
            ip, gpus = current_node_ip(), current_gpu_ids()
        except Exception:  # noqa: BLE001
            ip, gpus = "local", []
        return {"worker_id": self.worker_id, "node_ip": ip, "gpu_ids": gpus,
                "policy_version": self._policy_version}

    def _result(self, request, chunk, output=None, error=None) -> RayChunkResult:
        return RayChunkResult(request_id=request.request_id, worker_id=self.worker_id, chunk=chunk,
                              output=output, metrics=self.worker_metadata(),
                              policy_version=self._policy_version, error=error)

    def execute_chunk(self, request: GenerationRequest, chunk: MicroBatchPlan) -> RayChunkResult:
        self.load_policy()
        want = request.policy_version
        if want is not None and self._policy_version != want:
            return self._result(request, chunk, error=(
                f"policy_version mismatch: expected={want}, actual={self._policy_version}"))
        try:
            out = self.executor.forward_chunk(request, chunk)
            return self._result(request, chunk, output=to_cpu(out) if self.transfer == "cpu" else out)
        except Exception as exc:  # noqa: BLE001 - reported to the driver
            return self._result(request, chunk, error=str(exc))


__all__ = ["RayRolloutWorker", "build_executor_from_spec", "to_cpu"]
