"""Details of the family registry that other layers lean on: registration order, aliases, the
collector registry being derived from it, and which sampling fields a family's request declares
(reference expectations: ``tests/rollouts/test_family_registry.py``)."""

import pytest

from visionrl_b200.rollouts.collector import COLLECTOR_REGISTRY
from visionrl_b200.rollouts.collector import configs as C
from visionrl_b200.rollouts.families.specs import (DIFFUSION_COMMON_SAMPLING_FIELDS, DIFFUSION_RETURN_ARTIFACTS,
                                                   DIFFUSION_VIDEO_SAMPLING_FIELDS, FAMILY_REGISTRY,
                                                   get_rollout_family_entry, normalize_rollout_family,
                                                   registered_rollout_families)

CONFIGS = {"sd3_5": C.SD3_5CollectorConfig, "wan_2_1": C.Wan_2_1CollectorConfig,
           "cosmos": C.CosmosPredict2CollectorConfig, "janus_pro": C.JanusProCollectorConfig,
           "nextstep_1": C.NextStep1CollectorConfig}


def test_families_are_registered_in_a_fixed_order_with_their_config_classes():
    assert registered_rollout_families() == ("sd3_5", "wan_2_1", "cosmos", "janus_pro", "nextstep_1")
    for family, cls in CONFIGS.items():
        entry = FAMILY_REGISTRY[family]
        assert entry.family == family and entry.task
        assert entry.collector.config_cls.endswith(f":{cls.__name__}")
        assert ":" in entry.gatherer.import_path and ":" in entry.executor_cls and ":" in entry.runtime_builder


@pytest.mark.parametrize("alias,expected", [("wan", "wan_2_1"), ("cosmos_predict2", "cosmos"),
                                            ("janus", "janus_pro"), ("nextstep", "nextstep_1")])
def test_aliases_resolve_to_the_canonical_entry(alias, expected):
    assert normalize_rollout_family(alias) == expected
    assert get_rollout_family_entry(alias) is FAMILY_REGISTRY[expected]


def test_collector_registry_is_derived_from_the_family_registry():
    assert set(COLLECTOR_REGISTRY) == set(FAMILY_REGISTRY)
    for family, entry in FAMILY_REGISTRY.items():
        collector = COLLECTOR_REGISTRY[family]
        assert (collector.family, collector.task, collector.kind) == (entry.family, entry.task, entry.collector.kind)
        assert collector.config_cls is CONFIGS[family]


def test_diffusion_families_declare_their_request_shape():
    assert FAMILY_REGISTRY["sd3_5"].collector.sampling_fields == DIFFUSION_COMMON_SAMPLING_FIELDS
    assert FAMILY_REGISTRY["wan_2_1"].collector.sampling_fields == DIFFUSION_VIDEO_SAMPLING_FIELDS
    assert FAMILY_REGISTRY["cosmos"].collector.sampling_fields == (*DIFFUSION_VIDEO_SAMPLING_FIELDS, "fps")
    for family in ("sd3_5", "wan_2_1", "cosmos"):
        collector = FAMILY_REGISTRY[family].collector
        assert {"noise_level", "sde_type", "return_kl"} <= set(collector.sampling_fields)
        assert collector.return_artifacts == DIFFUSION_RETURN_ARTIFACTS


def test_unknown_family_is_a_clear_error():
    with pytest.raises(ValueError, match="unsupported rollout family"):
        get_rollout_family_entry("not_a_family")
