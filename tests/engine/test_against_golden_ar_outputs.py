"""Autoregressive helpers, packers and token evaluators against recorded outputs of the reference's
own code for the calls of ``golden_ar_cases.compute``."""

import os

import pytest
import torch

from tests.engine.golden_ar_cases import compute

GOLDEN = torch.load(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "ar_path_outputs.pt"))


@pytest.fixture(scope="module")
def outputs():
    return compute()


def test_every_recorded_value_is_computed(outputs):
    assert set(outputs) == set(GOLDEN) and len(GOLDEN) > 70


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_value_matches_the_recorded_one(outputs, key):
    got, want = outputs[key].detach().float(), GOLDEN[key].float()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), (key, float((got - want).abs().max()))
