"""Collector configuration defaults and built generation requests of all five families against
what the reference's collectors produce (``golden_request_cases.compute``)."""

import json
import os

import pytest

from tests.rollouts.golden_request_cases import compute

with open(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "collector_requests.json")) as fh:
    GOLDEN = json.load(fh)


@pytest.fixture(scope="module")
def outputs():
    return compute()


def test_every_family_is_covered(outputs):
    assert set(outputs) == set(GOLDEN) and len(GOLDEN) == 15
    assert {k.split("/")[0] for k in GOLDEN} == {"sd3_5", "wan_2_1", "cosmos", "janus_pro", "nextstep_1"}


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_request_or_config_matches(outputs, key):
    assert json.loads(outputs[key]) == json.loads(GOLDEN[key])
