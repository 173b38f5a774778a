"""Model names and where their policy classes live.

Entries are ``"package.module:Class"`` strings, imported on first use and then remembered, so
listing or registering models never imports a model family (and its kernels) that the run does not
touch.  The names are the ones configs use (``vrl/models/registry.py:7-30`` keeps the same table
for the reference's adapters; here every entry points at a native policy of this package).
"""

from __future__ import annotations

import importlib

_FAMILIES = "visionrl_b200.models.families"
_LOCATIONS: dict[str, str] = {
    "sd3_5-native-t2i": f"{_FAMILIES}.sd3_5.policy:SD3_5Policy",
    "sd3_5-diffusers-t2i": f"{_FAMILIES}.sd3_5.policy:SD3_5Policy",
    "wan-native-t2v": f"{_FAMILIES}.wan_2_1.diffusers_policy:WanT2VDiffusersPolicy",
    "wan-diffusers-t2v": f"{_FAMILIES}.wan_2_1.diffusers_policy:WanT2VDiffusersPolicy",
    "wan-official-t2v": f"{_FAMILIES}.wan_2_1.official_policy:WanT2VOfficialPolicy",
    "cosmos-predict2": f"{_FAMILIES}.cosmos.policy:CosmosPredict2Policy",
    "janus-pro": f"{_FAMILIES}.janus_pro.policy:JanusProPolicy",
    "nextstep-1": f"{_FAMILIES}.nextstep_1.policy:NextStep1Policy",
}
_LOADED: dict[str, type] = {}


def register_model(name: str, spec: str) -> None:
    """Add or replace an entry; ``spec`` is ``"package.module:Class"``."""
    module_path, sep, cls_name = spec.rpartition(":")
    if not (sep and module_path and cls_name):
        raise ValueError(f"model spec for {name!r} must look like 'package.module:Class', got {spec!r}")
    _LOCATIONS[name] = spec
    _LOADED.pop(name, None)


def resolve_model(name: str) -> type:
    cls = _LOADED.get(name)
    if cls is None:
        if name not in _LOCATIONS:
            raise KeyError(f"unknown model {name!r}; known: {', '.join(list_models())}")
        module_path, _, cls_name = _LOCATIONS[name].rpartition(":")
        cls = _LOADED[name] = getattr(importlib.import_module(module_path), cls_name)
    return cls


def list_models() -> list[str]:
    return sorted(_LOCATIONS)
