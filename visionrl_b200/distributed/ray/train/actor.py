"""Trainer-owning actor: the trainer is built inside the actor from a
``trainer_factory`` (callable or import path), never on the driver
(reference: ``vrl/distributed/ray/train/actor.py:15-114``)."""

from __future__ import annotations

import asyncio
import inspect
import threading
from typing import Any

from visionrl_b200.distributed.ray.dependencies import current_gpu_ids, current_node_ip
from visionrl_b200.distributed.ray.module_loading import import_from_path


def _get(cfg: Any, key: str, default: Any = None) -> Any:
    return cfg.get(key, default) if isinstance(cfg, dict) else getattr(cfg, key, default)


def run_awaitable(result: Any) -> Any:
    """Resolve ``result`` whether or not an event loop is already running."""
    if not inspect.isawaitable(result):
        return result
    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(result)
    box: dict[str, Any] = {}

    def target() -> None:
        try:
            box["value"] = asyncio.run(result)
        except BaseException as exc:  # noqa: BLE001
            box["error"] = exc

    t = threading.Thread(target=target, daemon=True)
    t.start()
    t.join()
    if "error" in box:
        raise box["error"]
    return box["value"]


class RayTrainActor:
    def __init__(self, train_config: Any | None = None) -> None:
        self.train_config = train_config
        self.trainer: Any | None = None

    def setup(self, train_config: Any | None = None) -> None:
        if train_config is not None:
            self.train_config = train_config
        if self.train_config is None:
            raise ValueError("RayTrainActor.setup requires train_config")
        factory = _get(self.train_config, "trainer_factory")
        if factory is None:
            raise NotImplementedError(
                "RayTrainActor requires `trainer_factory` in train_config; the driver must not "
                "construct CUDA trainer objects itself")
        if isinstance(factory, str):
            factory = import_from_path(factory)
        if not callable(factory):
            raise TypeError("trainer_factory must be callable or an import path")
        params = inspect.signature(factory).parameters
        if "train_config" in params or any(p.kind is p.VAR_KEYWORD for p in params.values()):
            self.trainer = factory(train_config=self.train_config)
        elif any(p.default is p.empty and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)
                 for p in params.values()):
            self.trainer = factory(self.train_config)
        else:
            self.trainer = factory()

    def train_step(self, prompt_batch: list[Any]) -> Any:
        if self.trainer is None:
            self.setup()
        return run_awaitable(self.trainer.step(prompt_batch))

    def metadata(self) -> dict[str, Any]:
        try:
            ip, gpus = current_node_ip(), current_gpu_ids()
        except Exception:  # noqa: BLE001
            ip, gpus = "local", []
        return {"node_ip": ip, "gpu_ids": gpus, "trainer_loaded": self.trainer is not None}


__all__ = ["RayTrainActor", "run_awaitable"]
