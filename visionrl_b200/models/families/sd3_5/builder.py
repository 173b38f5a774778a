"""SD3.5 family builder: config → ``RuntimeBuildSpec`` → ``RuntimeBundle``."""

from __future__ import annotations

from typing import Any

from visionrl_b200.models.families.common_builder import (
    build_diffusion_runtime_bundle, extract_diffusion_runtime_spec,
)
from visionrl_b200.models.runtime import RuntimeBuildSpec, RuntimeBundle

_ADAPTER_BY_BACKEND = {
    "native": "visionrl_b200.models.families.sd3_5.policy:SD3_5Policy",
    "diffusers": "visionrl_b200.models.families.sd3_5.policy:SD3_5Policy",
}
_CAPS = {"supports_stepwise": True, "supports_cfg": True, "supports_batched_decode": True,
         "supports_reference_conditioning": False}


def extract_sd3_5_runtime_spec(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBuildSpec:
    return extract_diffusion_runtime_spec(cfg, device, weight_dtype, task_variant="t2i")


def build_sd3_5_runtime_bundle(spec: RuntimeBuildSpec) -> RuntimeBundle:
    return build_diffusion_runtime_bundle(spec, _ADAPTER_BY_BACKEND, family="sd3_5", caps=_CAPS)


def build_sd3_5_runtime_bundle_from_cfg(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBundle:
    return build_sd3_5_runtime_bundle(extract_sd3_5_runtime_spec(cfg, device, weight_dtype))
