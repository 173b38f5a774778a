"""The serialisable rollout runtime spec each experiment produces, against what the reference's
``build_rollout_runtime_inputs`` produces from the same YAML (``tests/golden/runtime_specs.json``).
Four entries are this package's own by design and are left out of the comparison: the backend
preference and the native shape block (models are built natively, not through an external pipeline)
and the two import paths (they name this package's builder and executor)."""

import json
import os

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.rollouts.runtime.launch_inputs import build_rollout_runtime_inputs

with open(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "runtime_specs.json")) as fh:
    GOLDEN = json.load(fh)
OWN = ("backend_preference", "native_backend_config", "executor_cls", "runtime_builder")
FAMILY = {"sd3_5_ocr_grpo": "sd3_5", "wan_2_1_1_3b_grpo": "wan_2_1", "wan_2_1_14b_grpo": "wan_2_1",
          "cosmos_predict2_2b_grpo": "cosmos", "janus_pro_1b_grpo": "janus_pro", "nextstep_1_ocr_grpo": "nextstep_1"}


def _clean(obj):
    if isinstance(obj, dict):
        return {str(k): (sorted(v) if k == "target_modules" and isinstance(v, (list, tuple)) else _clean(v))
                for k, v in obj.items() if k not in OWN}
    if isinstance(obj, (list, tuple)):
        return [_clean(v) for v in obj]
    if isinstance(obj, (set, frozenset)):
        return sorted(_clean(v) for v in obj)
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return str(obj)


@pytest.mark.parametrize("experiment", sorted(GOLDEN))
def test_spec_matches_the_recorded_one(experiment):
    cfg = load_config(f"experiment/{experiment}")
    inputs = build_rollout_runtime_inputs(cfg, FAMILY[experiment], weight_dtype=torch.bfloat16, policy_version=4)
    got = _clean({"spec": inputs.runtime_spec.to_dict(), "gatherer": type(inputs.gatherer).__name__})
    assert got == GOLDEN[experiment]
