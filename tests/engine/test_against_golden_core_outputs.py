"""Engine core, micro-batching, the averaged-parameter wrapper, the reward mix and batch stacking
against what the reference's own code gives for the calls of ``golden_core_cases.compute``."""

import json
import math
import os

import pytest

from tests.engine.golden_core_cases import compute

with open(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "engine_core_outputs.json")) as fh:
    GOLDEN = json.load(fh)


def _same(a, b) -> bool:
    if isinstance(a, float) or isinstance(b, float):
        return isinstance(a, (int, float)) and isinstance(b, (int, float)) and math.isclose(a, b, rel_tol=1e-5, abs_tol=1e-6)
    if isinstance(a, list) and isinstance(b, list):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, dict) and isinstance(b, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    return a == b


@pytest.fixture(scope="module")
def outputs():
    return compute()


def test_every_recorded_case_is_computed(outputs):
    assert set(outputs) == set(GOLDEN) and len(GOLDEN) >= 24


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_result_matches_the_recorded_one(outputs, key):
    assert _same(json.loads(outputs[key]), json.loads(GOLDEN[key])), (outputs[key][:300], GOLDEN[key][:300])
