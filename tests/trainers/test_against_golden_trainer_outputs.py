"""``OnlineTrainer.step`` against recorded outputs of the reference's trainer for the fixed runs of
``golden_trainer_cases.compute``: every metric of both steps in three set-ups, the order of the
evaluated timesteps, the parameters after four clipped optimiser steps, the averaged (EMA)
parameters and the step counters."""

import os

import pytest
import torch

from tests.trainers.golden_trainer_cases import compute

GOLDEN = torch.load(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "trainer_outputs.pt"))


@pytest.fixture(scope="module")
def outputs():
    return compute()


def test_every_recorded_value_is_computed(outputs):
    assert set(outputs) == set(GOLDEN) and len(GOLDEN) > 100
    assert any(k.endswith("/ema/0") for k in GOLDEN) and any("/param/" in k for k in GOLDEN)


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_value_matches_the_recorded_one(outputs, key):
    got, want = outputs[key].detach().float(), GOLDEN[key].float()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), (key, float((got - want).abs().max()))
