"""The algorithm layer against recorded outputs of the reference implementation's own functions for
the fixed calls of ``golden_cases.compute`` (105 tensors: preference loss and its statistics, group
advantages, clipped losses with both KL forms, the token-level loss with both estimators, the SDE
and CPS steps including the sampled values for a given generator, replayed log-probabilities, the
deterministic path, the statistics tracker, OCR distances, the K-repeat sampler's index order)."""

import os

import pytest
import torch

from tests.algorithms.golden_cases import compute

GOLDEN = torch.load(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "algorithm_outputs.pt"))


@pytest.fixture(scope="module")
def outputs():
    return compute()


def test_every_recorded_case_is_computed(outputs):
    assert set(outputs) == set(GOLDEN) and len(GOLDEN) >= 100


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_output_matches_the_recorded_value(outputs, key):
    got, want = outputs[key].detach().float(), GOLDEN[key].float()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), float((got - want).abs().max())
