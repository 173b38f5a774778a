"""Executor -> packer -> evaluator against recorded outputs of the reference's own classes for the
stub policy and the six sampling set-ups of ``golden_pipeline_cases.compute`` (282 tensors:
trajectories, log-probabilities, KL records, decoded outputs, sample order, packed batches,
replayed signals with the adapter-off reference)."""

import os

import pytest
import torch

from tests.engine.golden_pipeline_cases import compute

GOLDEN = torch.load(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "rollout_pipeline_outputs.pt"))


@pytest.fixture(scope="module")
def outputs():
    return compute()


def test_every_recorded_value_is_computed(outputs):
    assert set(outputs) == set(GOLDEN) and len(GOLDEN) > 250
    for case in ("base", "kl", "cps", "window", "same", "nlow"):
        assert f"{case}/traj.rollout_log_probs" in GOLDEN and f"{case}/sig0.log_prob" in GOLDEN


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_value_matches_the_recorded_one(outputs, key):
    got, want = outputs[key].detach().float(), GOLDEN[key].float()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), (key, float((got - want).abs().max()))
