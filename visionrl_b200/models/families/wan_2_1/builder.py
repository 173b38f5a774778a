"""Wan-2.1 family builder."""

from __future__ import annotations

from typing import Any

from visionrl_b200.models.families.common_builder import (
    build_diffusion_runtime_bundle, extract_diffusion_runtime_spec,
)
from visionrl_b200.models.runtime import RuntimeBuildSpec, RuntimeBundle

_ADAPTER_BY_BACKEND = {
    "native": "visionrl_b200.models.families.wan_2_1.diffusers_policy:WanT2VDiffusersPolicy",
    "diffusers": "visionrl_b200.models.families.wan_2_1.diffusers_policy:WanT2VDiffusersPolicy",
    "official": "visionrl_b200.models.families.wan_2_1.official_policy:WanT2VOfficialPolicy",
}
_CAPS = {"supports_stepwise": True, "supports_cfg": True, "supports_batched_decode": True,
         "supports_reference_conditioning": False, "supports_sequence_parallel": True}


def extract_wan_2_1_runtime_spec(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBuildSpec:
    return extract_diffusion_runtime_spec(cfg, device, weight_dtype, task_variant="t2v")


def build_wan_2_1_runtime_bundle(spec: RuntimeBuildSpec) -> RuntimeBundle:
    return build_diffusion_runtime_bundle(spec, _ADAPTER_BY_BACKEND, family="wan_2_1", caps=_CAPS)


def build_wan_2_1_runtime_bundle_from_cfg(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBundle:
    return build_wan_2_1_runtime_bundle(extract_wan_2_1_runtime_spec(cfg, device, weight_dtype))
