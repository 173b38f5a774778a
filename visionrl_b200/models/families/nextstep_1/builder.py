"""NextStep-1 family builder (reference: ``vrl/models/families/nextstep_1/builder.py:11-126``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.config.node import to_container
from visionrl_b200.models.runtime import RuntimeBuildSpec, RuntimeBundle
from visionrl_b200.rollouts.runtime.config import cfg_path


def extract_nextstep_1_runtime_spec(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBuildSpec:
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
        "vae_path": str(cfg_path(cfg, "model.vae_path", "") or ""),
        "freeze_image_head": bool(cfg_path(cfg, "model.freeze_image_head", False)),
        "sampling": {
            "cfg_scale": float(cfg.sampling.cfg_scale),
            "num_flow_steps": int(cfg.sampling.num_flow_steps),
            "noise_level": float(cfg_path(cfg, "rollout.noise_level",
                                          cfg_path(cfg, "sampling.noise_level", 1.0))),
            "image_token_num": int(cfg.sampling.image_token_num),
            "image_size": int(cfg.sampling.image_size),
        },
    }
    # the same facts in the two places the reference's spec carries them
    return RuntimeBuildSpec(
        model_name_or_path=str(model.path), device=device,
        dtype=cfg_path(cfg, "model.dtype", None) or weight_dtype, backend_preference=("native",),
        task_variant="ar_t2i", use_lora=bool(model.use_lora), lora_config=lora_cfg,
        scheduler_config=dict(native["sampling"]), native_backend_config=native,
        extra={"vae_path": native["vae_path"], "freeze_image_head": native["freeze_image_head"],
               "freeze_vae": bool(cfg_path(cfg, "model.freeze_vae", True)),
               "gradient_checkpointing": bool(cfg_path(cfg, "actor.gradient_checkpointing", False))})


def _nextstep_1_config_from_runtime_spec(spec: RuntimeBuildSpec):
    from visionrl_b200.models.families.nextstep_1.policy import NextStep1Config

    native = dict(spec.native_backend_config or {})
    extra = dict(spec.extra or {})
    sampling = {**dict(spec.scheduler_config or {}), **dict(native.get("sampling") or {})}
    native.setdefault("vae_path", extra.get("vae_path", ""))
    native.setdefault("freeze_image_head", extra.get("freeze_image_head", False))
    lora = dict(spec.lora_config or {})
    return NextStep1Config(
        model_path=spec.model_name_or_path, vae_path=str(native.get("vae_path", "")),
        dtype=str(spec.dtype).removeprefix("torch."), use_lora=bool(spec.use_lora),
        lora_rank=int(lora.get("rank", 32)), lora_alpha=int(lora.get("alpha", 64)),
        lora_dropout=float(lora.get("dropout", 0.0)), lora_init=str(lora.get("init", "gaussian")),
        lora_target_modules=tuple(lora.get("target_modules", ("q_proj", "k_proj", "v_proj", "o_proj"))),
        cfg_scale=float(sampling.get("cfg_scale", 4.5)),
        num_flow_steps=int(sampling.get("num_flow_steps", 20)),
        noise_level=float(sampling.get("noise_level", 1.0)),
        image_token_num=int(sampling.get("image_token_num", 1024)),
        image_size=int(sampling.get("image_size", 256)),
        freeze_image_head=bool(native.get("freeze_image_head", False)),
        random_init=bool(native.get("random_init", True)), init_seed=int(native.get("init_seed", 0)),
        arch=dict(native.get("arch") or {}), freeze_vae=bool(extra.get("freeze_vae", True)),
        gradient_checkpointing=bool(extra.get("gradient_checkpointing", False)))


def build_nextstep_1_runtime_bundle(spec: RuntimeBuildSpec) -> RuntimeBundle:
    from visionrl_b200.models.families.nextstep_1.policy import NextStep1Policy

    policy = NextStep1Policy(_nextstep_1_config_from_runtime_spec(spec), device=spec.device)
    return RuntimeBundle(
        policy=policy, trainable_modules=policy.trainable_modules, scheduler=None,
        backend_kind="native", backend_handle=policy,
        runtime_caps={"supports_stepwise": True, "supports_cfg": True, "supports_token_scheduler": True},
        metadata={"model_path": spec.model_name_or_path, "task_variant": spec.task_variant,
                  "dtype": str(spec.dtype), "use_lora": spec.use_lora, "family": "nextstep_1"})


def build_nextstep_1_runtime_bundle_from_cfg(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBundle:
    return build_nextstep_1_runtime_bundle(extract_nextstep_1_runtime_spec(cfg, device, weight_dtype))
