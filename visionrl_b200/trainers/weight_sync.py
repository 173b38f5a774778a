"""Trainer → rollout weight synchronisation front-ends
(reference: ``vrl/trainers/weight_sync.py:11-108``).

``RayRuntimeWeightSyncer`` ships a CPU copy of the state with a monotonically
increasing policy version (the reference's data path).  ``DeviceWeightSyncer`` is
the B200 path: tensors stay on the GPU and the runtime applies them device-to-device
(or does nothing when rollout and trainer share one copy), only the version moves.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any


class WeightSyncer(ABC):
    @abstractmethod
    async def push(self, state_dict: dict[str, Any]) -> None: ...

    @abstractmethod
    async def pull(self) -> dict[str, Any]: ...


class InMemoryWeightSyncer(WeightSyncer):
    def __init__(self) -> None:
        self._state: dict[str, Any] = {}

    async def push(self, state_dict: dict[str, Any]) -> None:
        self._state = dict(state_dict)

    async def pull(self) -> dict[str, Any]:
        return dict(self._state)


def _cpu_copy(value: Any) -> Any:
    if hasattr(value, "detach") and hasattr(value, "cpu"):
        return value.detach().cpu()
    if isinstance(value, dict):
        return {k: _cpu_copy(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_cpu_copy(v) for v in value)
    return value


class RayRuntimeWeightSyncer(WeightSyncer):
    def __init__(self, runtime: Any, *, initial_policy_version: int | None = None) -> None:
        self.runtime = runtime
        current = initial_policy_version
        if current is None:
            current = getattr(runtime, "current_policy_version", None)
        self.policy_version = int(current or 0)
        self._last: dict[str, Any] = {}

    def _next_version(self) -> int:
        self.policy_version += 1
        return self.policy_version

    async def push(self, state_dict: dict[str, Any]) -> None:
        state = _cpu_copy(dict(state_dict))
        self._last = state
        await self.runtime.update_weights(state, self._next_version())

    async def pull(self) -> dict[str, Any]:
        return dict(self._last)


class DeviceWeightSyncer(RayRuntimeWeightSyncer):
    """Versioned push without a host round trip."""

    def __init__(self, runtime: Any, *, initial_policy_version: int | None = None,
                 trainable_only: bool = True) -> None:
        super().__init__(runtime, initial_policy_version=initial_policy_version)
        self.trainable_only = trainable_only

    async def push(self, state_dict: dict[str, Any]) -> None:
        version = self._next_version()
        if getattr(self.runtime, "shares_trainer_weights", False):
            await self.runtime.update_weights(None, version)
            return
        self._last = dict(state_dict)
        await self.runtime.update_weights(self._last, version)


def build_runtime_weight_syncer(runtime: Any, *, initial_policy_version: int | None = None):
    """A syncer exists only if the runtime can receive weights and has sync enabled."""
    if not callable(getattr(runtime, "update_weights", None)):
        return None
    if getattr(runtime, "weight_sync", None) is None:
        return None
    if hasattr(runtime, "shares_trainer_weights"):
        return DeviceWeightSyncer(runtime, initial_policy_version=initial_policy_version)
    return RayRuntimeWeightSyncer(runtime, initial_policy_version=initial_policy_version)
