"""Cosmos-Predict2 family builder."""

from __future__ import annotations

from typing import Any

from visionrl_b200.models.families.common_builder import (
    build_diffusion_runtime_bundle, extract_diffusion_runtime_spec,
)
from visionrl_b200.models.runtime import RuntimeBuildSpec, RuntimeBundle

_ADAPTER_BY_BACKEND = {
    "native": "visionrl_b200.models.families.cosmos.policy:CosmosPredict2Policy",
    "diffusers": "visionrl_b200.models.families.cosmos.policy:CosmosPredict2Policy",
}
_CAPS = {"supports_stepwise": True, "supports_cfg": True, "supports_batched_decode": True,
         "supports_reference_conditioning": True}


def extract_cosmos_predict2_runtime_spec(cfg: Any, device: Any, weight_dtype: Any) -> RuntimeBuildSpec:
    return extract_diffusion_runtime_spec(cfg, device, weight_dtype, task_variant="video2world")


def build_cosmos_predict2_runtime_bundle(spec: RuntimeBuildSpec) -> RuntimeBundle:
    bundle = build_diffusion_runtime_bundle(spec, _ADAPTER_BY_BACKEND, family="cosmos", caps=_CAPS)
    ref = (spec.extra or {}).get("reference_image")
    if ref:
        bundle.policy.set_reference_image(ref)
    return bundle


def build_cosmos_predict2_runtime_bundle_from_cfg(cfg: Any, device: Any,
                                                  weight_dtype: Any) -> RuntimeBundle:
    return build_cosmos_predict2_runtime_bundle(
        extract_cosmos_predict2_runtime_spec(cfg, device, weight_dtype))
