"""Janus-Pro family builder (reference: ``vrl/models/families/janus_pro/builder.py:11-113``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.config.node import to_container
from visionrl_b200.models.runtime import RuntimeBuildSpec, RuntimeBundle
from visionrl_b200.rollouts.runtime.config import cfg_path


def extract_janus_pro_runtime_spec(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBuildSpec:
    model = cfg.model
    lora_cfg = None
    if bool(model.use_lora):
        lora_cfg = {"rank": int(model.lora.rank), "alpha": int(model.lora.alpha),
                    "dropout": float(cfg_path(cfg, "model.lora.dropout", 0.0)),
                    "init": str(cfg_path(cfg, "model.lora.init", "gaussian")),
                    "target_modules": list(model.lora.target_modules)}
    native = {
        "arch": to_container(cfg_path(cfg, "model.arch", {}) or {}),
        "random_init": bool(cfg_path(cfg, "model.random_init", False)),
        "init_seed": int(cfg_path(cfg, "model.init_seed", 0) or 0),
        "int4_decode": bool(cfg_path(cfg, "model.int4_decode", False)),
        "sampling": {
            "cfg_weight": float(cfg.sampling.cfg_weight),
            "temperature": float(cfg_path(cfg, "sampling.temperature",
                                          cfg_path(cfg, "rollout.temperature", 1.0))),
            "image_token_num": int(cfg.sampling.image_token_num),
            "image_size": int(cfg.sampling.image_size),
        },
        "freeze_vq": bool(cfg_path(cfg, "model.freeze_vq", True)),
    }
    # the same facts in the two places the reference's spec carries them (sampling defaults under
    # ``scheduler_config``, freeze switches under ``extra``), so a spec written either way builds
    sampling = native["sampling"]
    return RuntimeBuildSpec(
        model_name_or_path=str(model.path), device=device,
        dtype=cfg_path(cfg, "model.dtype", None) or weight_dtype, backend_preference=("native",),
        task_variant="ar_t2i", use_lora=bool(model.use_lora), lora_config=lora_cfg,
        scheduler_config={"cfg_weight": sampling["cfg_weight"], "image_token_num": sampling["image_token_num"],
                          "temperature": sampling["temperature"]},
        native_backend_config=native,
        extra={"freeze_vq": native["freeze_vq"],
               "freeze_vision_encoder": bool(cfg_path(cfg, "model.freeze_vision_encoder", True)),
               "freeze_aligner": bool(cfg_path(cfg, "model.freeze_aligner", True))})


def _janus_config_from_runtime_spec(spec: RuntimeBuildSpec):
    from visionrl_b200.models.families.janus_pro.policy import JanusProConfig

    native = dict(spec.native_backend_config or {})
    extra = dict(spec.extra or {})
    sampling = {**dict(spec.scheduler_config or {}), **dict(native.get("sampling") or {})}
    native.setdefault("freeze_vq", extra.get("freeze_vq", True))
    lora = dict(spec.lora_config or {})
    dtype = str(spec.dtype).removeprefix("torch.")
    image_size = int(sampling.get("image_size", 384))
    tokens = int(sampling.get("image_token_num", 576))
    side = max(1, int(round(tokens ** 0.5)))
    return JanusProConfig(
        model_path=spec.model_name_or_path, dtype=dtype, use_lora=bool(spec.use_lora),
        lora_rank=int(lora.get("rank", 128)), lora_alpha=int(lora.get("alpha", 256)),
        lora_dropout=float(lora.get("dropout", 0.0)), lora_init=str(lora.get("init", "gaussian")),
        lora_target_modules=tuple(lora.get("target_modules", ("q_proj", "k_proj", "v_proj", "o_proj"))),
        cfg_weight=float(sampling.get("cfg_weight", 5.0)),
        temperature=float(sampling.get("temperature", 1.0)), image_token_num=tokens,
        image_size=image_size, patch_size=max(1, image_size // side),
        freeze_vq=bool(native.get("freeze_vq", True)), random_init=bool(native.get("random_init", True)),
        init_seed=int(native.get("init_seed", 0)), int4_decode=bool(native.get("int4_decode", False)),
        arch=dict(native.get("arch") or {}),
        freeze_vision_encoder=bool(extra.get("freeze_vision_encoder", True)),
        freeze_aligner=bool(extra.get("freeze_aligner", True)))


def build_janus_pro_runtime_bundle(spec: RuntimeBuildSpec) -> RuntimeBundle:
    from visionrl_b200.models.families.janus_pro.policy import JanusProPolicy

    policy = JanusProPolicy(_janus_config_from_runtime_spec(spec), device=spec.device)
    return RuntimeBundle(
        policy=policy, trainable_modules=policy.trainable_modules, scheduler=None,
        backend_kind="native", backend_handle=policy,
        runtime_caps={"supports_stepwise": True, "supports_cfg": True, "supports_token_scheduler": True},
        metadata={"model_path": spec.model_name_or_path, "task_variant": spec.task_variant,
                  "dtype": str(spec.dtype), "use_lora": spec.use_lora, "family": "janus_pro"})


def build_janus_pro_runtime_bundle_from_cfg(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBundle:
    return build_janus_pro_runtime_bundle(extract_janus_pro_runtime_spec(cfg, device, weight_dtype))
