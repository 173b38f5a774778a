"""Lazy ``name → "module:Class"`` model registry (reference: ``vrl/models/registry.py:7-30``)."""

from __future__ import annotations

import importlib

_REGISTRY: dict[str, str] = {
    "sd3_5-native-t2i": "visionrl_b200.models.families.sd3_5.policy:SD3_5Policy",
    "sd3_5-diffusers-t2i": "visionrl_b200.models.families.sd3_5.policy:SD3_5Policy",
    "wan-native-t2v": "visionrl_b200.models.families.wan_2_1.diffusers_policy:WanT2VDiffusersPolicy",
    "wan-diffusers-t2v": "visionrl_b200.models.families.wan_2_1.diffusers_policy:WanT2VDiffusersPolicy",
    "wan-official-t2v": "visionrl_b200.models.families.wan_2_1.official_policy:WanT2VOfficialPolicy",
    "cosmos-predict2": "visionrl_b200.models.families.cosmos.policy:CosmosPredict2Policy",
    "janus-pro": "visionrl_b200.models.families.janus_pro.policy:JanusProPolicy",
    "nextstep-1": "visionrl_b200.models.families.nextstep_1.policy:NextStep1Policy",
}


def resolve_model(name: str) -> type:
    module_path, cls_name = _REGISTRY[name].rsplit(":", 1)
    return getattr(importlib.import_module(module_path), cls_name)


def register_model(name: str, spec: str) -> None:
    _REGISTRY[name] = spec


def list_models() -> list[str]:
    return sorted(_REGISTRY)
