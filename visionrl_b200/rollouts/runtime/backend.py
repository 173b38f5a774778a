"""Rollout backend construction from config
(reference: ``vrl/rollouts/runtime/backend.py:11-222``).

A driver that already holds the rollout policy on a CUDA device is rejected unless
``allow_driver_gpu_overlap`` is set — the default deployment keeps the driver's copy
off the rollout GPUs.  ``release_after_collect`` wraps the runtime so its workers
are torn down between collect phases and relaunched (with the last pushed weights
replayed) on the next ``generate``.
"""

from __future__ import annotations

from collections.abc import Iterable, Mapping
from typing import Any

from visionrl_b200.engine import RolloutBackend
from visionrl_b200.rollouts.runtime.config import RolloutBackendConfig, cfg_path

DRIVER_CUDA_OWNERSHIP_ERROR = (
    "Driver loaded rollout policy on CUDA. With the Ray-style backend set model.device=cpu so that the "
    "rollout workers own the CUDA copies, or set distributed.rollout.allow_driver_gpu_overlap=true "
    "for an explicitly colocated run."
)


def _is_cuda(device: Any) -> bool:
    kind = getattr(device, "type", None)
    return str(kind if kind is not None else device).lower().startswith("cuda")


def _device_of(obj: Any) -> tuple[bool, Any]:
    if obj is None:
        return False, None
    try:
        dev = obj.device
    except Exception:  # noqa: BLE001
        return False, None
    return (dev is not None), dev


def _param_devices(obj: Any, seen: set[int] | None = None) -> Iterable[Any]:
    if obj is None or isinstance(obj, (str, bytes)):
        return
    seen = seen if seen is not None else set()
    if id(obj) in seen:
        return
    seen.add(id(obj))
    if isinstance(obj, Mapping):
        for v in obj.values():
            yield from _param_devices(v, seen)
        return
    has, dev = _device_of(obj)
    if has:
        yield dev
        return
    params = getattr(obj, "parameters", None)
    if callable(params):
        for p in params():
            if getattr(p, "device", None) is not None:
                yield p.device
        return
    if isinstance(obj, Iterable):
        for v in obj:
            yield from _param_devices(v, seen)


def _driver_policy_on_cuda(driver_bundle, driver_policy, trainable_modules) -> bool:
    policy = driver_policy if driver_policy is not None else getattr(driver_bundle, "policy", None)
    has, dev = _device_of(policy)
    if has:
        return _is_cuda(dev)
    modules = trainable_modules
    if modules is None and driver_bundle is not None:
        modules = getattr(driver_bundle, "trainable_modules", None)
    return any(_is_cuda(d) for d in _param_devices(modules))


def validate_rollout_backend_config(cfg: Any, *, driver_bundle: Any | None = None,
                                    driver_policy: Any | None = None,
                                    trainable_modules: Any | None = None) -> RolloutBackendConfig:
    config = RolloutBackendConfig.from_cfg(cfg)
    if not config.allow_driver_gpu_overlap and _driver_policy_on_cuda(
            driver_bundle, driver_policy, trainable_modules):
        raise ValueError(DRIVER_CUDA_OWNERSHIP_ERROR)
    return config


def _launch(config: RolloutBackendConfig, runtime_spec: Any, gatherer: Any,
            driver_policy: Any | None = None) -> Any:
    if config.backend == "native":
        from visionrl_b200.distributed.native.runtime import NativeRolloutLauncher

        return NativeRolloutLauncher().launch(config.to_dict(), runtime_spec, gatherer,
                                              driver_policy=driver_policy)
    from visionrl_b200.distributed.ray.rollout.launcher import RayRolloutLauncher

    return RayRolloutLauncher().launch(config.to_dict(), runtime_spec, gatherer)


def build_rollout_backend_from_cfg(cfg: Any, *, driver_bundle: Any | None = None,
                                   driver_policy: Any | None = None,
                                   trainable_modules: Any | None = None,
                                   runtime_spec: Any | None = None,
                                   gatherer: Any | None = None) -> RolloutBackend:
    config = validate_rollout_backend_config(
        cfg, driver_bundle=driver_bundle, driver_policy=driver_policy,
        trainable_modules=trainable_modules)
    if runtime_spec is None:
        runtime_spec = cfg_path(cfg, "distributed.rollout.runtime_spec", None)
    if runtime_spec is None or gatherer is None:
        raise ValueError(
            "rollout backend requires runtime_spec plus gatherer so the launcher can construct "
            "workers through the runtime_builder+executor_cls path.")
    policy = driver_policy if driver_policy is not None else getattr(driver_bundle, "policy", None)
    if config.release_after_collect and config.backend == "ray":
        return ReleasableRayRolloutBackend(config, runtime_spec, gatherer)
    return _launch(config, runtime_spec, gatherer, policy)


def _spec_policy_version(runtime_spec: Any) -> int | None:
    try:
        from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec

        spec = GenerationRuntimeSpec.from_value(runtime_spec)
    except Exception:  # noqa: BLE001
        return None
    return None if spec.policy_version is None else int(spec.policy_version)


class ReleasableRayRolloutBackend(RolloutBackend):
    def __init__(self, config: RolloutBackendConfig, runtime_spec: Any, gatherer: Any) -> None:
        self.config, self.runtime_spec, self.gatherer = config, runtime_spec, gatherer
        self.weight_sync = object() if config.sync_trainable_state != "disabled" else None
        self.requires_driver_model_offload = config.gpus_per_worker > 0
        self.current_policy_version = _spec_policy_version(runtime_spec)
        self._runtime: Any | None = None
        self._last_state: Any | None = None

    async def _ensure_runtime(self) -> Any:
        if self._runtime is None:
            self._runtime = _launch(self.config, self.runtime_spec, self.gatherer)
            if self._last_state is not None:
                await self._runtime.update_weights(self._last_state,
                                                   int(self.current_policy_version))
        return self._runtime

    async def generate(self, request: Any) -> Any:
        return await (await self._ensure_runtime()).generate(request)

    async def update_weights(self, state_ref: Any, policy_version: int) -> None:
        if self.weight_sync is None:
            raise RuntimeError("ReleasableRayRolloutBackend has no rollout weight sync")
        self._last_state = state_ref
        self.current_policy_version = int(policy_version)
        if self._runtime is not None:
            await self._runtime.update_weights(state_ref, self.current_policy_version)

    async def release_memory(self) -> None:
        runtime, self._runtime = self._runtime, None
        if runtime is not None:
            await runtime.shutdown()

    async def shutdown(self) -> None:
        await self.release_memory()


__all__ = ["DRIVER_CUDA_OWNERSHIP_ERROR", "ReleasableRayRolloutBackend",
           "build_rollout_backend_from_cfg", "validate_rollout_backend_config"]
