"""Resource / backend selection of the rollout runtime
(reference: ``vrl/rollouts/runtime/config.py:9-107``).

``backend`` is ``"ray"`` (the reference's key, served here by in-process rollout
workers behind the same launcher names) or ``"native"`` (one rank per GPU under
``torch.distributed``, rollout colocated with the trainer shards).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

_MISSING = object()
_BACKENDS = ("ray", "native")
_SYNC_MODES = ("disabled", "lora_only", "full")


def cfg_get(node: Any, key: str, default: Any = None) -> Any:
    if node is None:
        return default
    getter = getattr(node, "get", None)
    if callable(getter):
        try:
            return getter(key, default)
        except TypeError:
            pass
    try:
        return node[key]
    except (KeyError, IndexError, TypeError):
        pass
    return getattr(node, key, default)


def cfg_path(cfg: Any, path: str, default: Any = None) -> Any:
    node = cfg
    for key in path.split("."):
        node = cfg_get(node, key, _MISSING)
        if node is _MISSING:
            return default
    return node


@dataclass(slots=True)
class RolloutBackendConfig:
    backend: str = "ray"
    num_workers: int = 1
    gpus_per_worker: float = 1.0
    cpus_per_worker: float = 1.0
    placement_strategy: str = "SPREAD"
    allow_driver_gpu_overlap: bool = False
    max_inflight_chunks_per_worker: int = 1
    sync_trainable_state: str = "disabled"
    release_after_collect: bool = False

    def __post_init__(self) -> None:
        if self.backend not in _BACKENDS:
            raise ValueError("backend must be 'ray' or 'native'")
        if self.num_workers < 1:
            raise ValueError("num_workers must be >= 1")
        if self.gpus_per_worker < 0:
            raise ValueError("gpus_per_worker must be >= 0")
        if self.cpus_per_worker <= 0:
            raise ValueError("cpus_per_worker must be > 0")
        if not self.placement_strategy:
            raise ValueError("placement_strategy must be non-empty")
        if self.max_inflight_chunks_per_worker < 1:
            raise ValueError("max_inflight_chunks_per_worker must be >= 1")
        if self.sync_trainable_state not in _SYNC_MODES:
            raise ValueError("sync_trainable_state must be 'disabled', 'lora_only' or 'full'")

    @classmethod
    def from_cfg(cls, cfg: Any) -> "RolloutBackendConfig":
        """Accepts a whole training config, its ``distributed`` node or a flat mapping."""
        if isinstance(cfg, cls):
            return cfg
        distributed = cfg_get(cfg, "distributed", _MISSING)
        if distributed is _MISSING:
            if cfg_get(cfg, "backend", _MISSING) is _MISSING:
                raise ValueError("distributed.backend or backend is required")
            distributed = cfg
        rollout = cfg_get(distributed, "rollout", _MISSING)
        if rollout is _MISSING:
            rollout = distributed
        backend = cfg_get(distributed, "backend", cfg_get(rollout, "backend", _MISSING))
        if backend is _MISSING:
            raise ValueError("distributed.backend or backend is required")

        def pick(key: str, default: Any) -> Any:
            value = cfg_get(rollout, key, _MISSING)
            if value is _MISSING:
                value = cfg_get(distributed, key, default)
            return value

        return cls(
            backend=str(backend), num_workers=int(pick("num_workers", 1)),
            gpus_per_worker=float(pick("gpus_per_worker", 1.0)),
            cpus_per_worker=float(pick("cpus_per_worker", 1.0)),
            placement_strategy=str(pick("placement_strategy", "SPREAD")),
            allow_driver_gpu_overlap=bool(pick("allow_driver_gpu_overlap", False)),
            max_inflight_chunks_per_worker=int(pick("max_inflight_chunks_per_worker", 1)),
            sync_trainable_state=str(pick("sync_trainable_state", "disabled")),
            release_after_collect=bool(pick("release_after_collect", False)),
        )

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


__all__ = ["RolloutBackendConfig", "cfg_get", "cfg_path"]
