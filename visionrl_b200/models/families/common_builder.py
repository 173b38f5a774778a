"""Spec extraction and bundle assembly shared by the diffusion family builders
(reference: ``vrl/models/families/sd3_5/builder.py:36-123`` and its Wan / Cosmos twins)."""

from __future__ import annotations

import importlib
import logging
from typing import Any

from visionrl_b200.config.node import to_container
from visionrl_b200.models.runtime import RuntimeBuildSpec, RuntimeBundle

logger = logging.getLogger(__name__)


def _get(node: Any, key: str, default: Any = None) -> Any:
    if node is None:
        return default
    if isinstance(node, dict):
        return node.get(key, default)
    return getattr(node, key, default)


def extract_diffusion_runtime_spec(cfg: Any, device: Any, weight_dtype: Any, *,
                                   task_variant: str) -> RuntimeBuildSpec:
    model = cfg.model
    lora_cfg = lora_path = None
    if model.use_lora:
        lora_path = _get(model.lora, "path") or None
        lora_cfg = {"rank": int(model.lora.rank), "alpha": int(model.lora.alpha),
                    "target_modules": list(model.lora.target_modules)}
    extra: dict[str, Any] = {}
    compile_cfg = _get(model, "torch_compile")
    if compile_cfg is not None and _get(compile_cfg, "enable"):
        extra["torch_compile"] = {"enable": True, "mode": _get(compile_cfg, "mode", "default")}
    ref_image = _get(model, "reference_image")
    if ref_image:
        extra["reference_image"] = ref_image
    native = {
        "arch": to_container(_get(model, "arch") or {}),
        "random_init": bool(_get(model, "random_init", False)),
        "init_seed": int(_get(model, "init_seed", 0) or 0),
        "decoder": to_container(_get(model, "decoder") or {}),
    }
    if _get(model, "shift") is not None:
        native["shift"] = float(model.shift)
    text_encoder = _get(model, "text_encoder")
    if text_encoder is not None and _get(text_encoder, "path"):
        # a local pipeline directory (text_encoder*/ + tokenizer*/): real prompt conditioning
        native["text_encoder_path"] = str(_get(text_encoder, "path"))
    return RuntimeBuildSpec(
        model_name_or_path=str(_get(model, "path", "")), device=device, dtype=weight_dtype,
        backend_preference=(str(_get(model, "backend", "native") or "native"),), task_variant=task_variant,
        use_lora=bool(model.use_lora), lora_path=lora_path, lora_config=lora_cfg,
        scheduler_config={"num_steps": int(cfg.sampling.num_steps)},
        native_backend_config=native, extra=extra,
    )


def build_diffusion_runtime_bundle(spec: RuntimeBuildSpec, adapters: dict[str, str], *,
                                   family: str, caps: dict[str, Any]) -> RuntimeBundle:
    backend = spec.backend_preference[0]
    if backend not in adapters:
        raise NotImplementedError(
            f"{family} has no adapter for backend={backend!r}; registered: {sorted(adapters)}")
    mod_path, cls_name = adapters[backend].rsplit(":", 1)
    adapter_cls = getattr(importlib.import_module(mod_path), cls_name)
    logger.info("Building %s runtime bundle (backend=%s)", family, backend)
    adapter = adapter_cls.from_spec(spec)
    if spec.use_lora:
        adapter.apply_lora(spec)
    else:
        adapter.enable_full_finetune()
    compile_cfg = (spec.extra or {}).get("torch_compile") or {}
    if compile_cfg.get("enable"):
        adapter.torch_compile_transformer(compile_cfg["mode"])
    steps = (spec.scheduler_config or {}).get("num_steps")
    if steps is not None:
        adapter.set_num_steps(steps)
    return RuntimeBundle(
        policy=adapter, trainable_modules=adapter.trainable_modules, scheduler=adapter.scheduler,
        backend_kind=backend, backend_handle=adapter.backend_handle, runtime_caps=dict(caps),
        metadata={"model_path": spec.model_name_or_path, "task_variant": spec.task_variant,
                  "dtype": str(spec.dtype), "use_lora": spec.use_lora},
    )
