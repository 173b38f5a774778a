"""TokenGRPO: masking, clip statistics and KL estimators."""

import math

import pytest
import torch

from vrl.algorithms import GRPO, GRPOConfig
from vrl.algorithms.grpo_token import TokenGRPO, TokenGRPOConfig
from vrl.rollouts.evaluators.types import SignalBatch


def test_advantages_identical_to_grpo():
    r, g = torch.tensor([1.0, 2.0, 4.0, 0.0]), torch.tensor([0, 0, 1, 1])
    a = TokenGRPO(TokenGRPOConfig()).compute_advantages_from_tensors(r, g)
    b = GRPO(GRPOConfig()).compute_advantages_from_tensors(r, g)
    assert torch.equal(a, b)


def test_full_zero_mask_gives_zero_loss():
    algo = TokenGRPO(TokenGRPOConfig())
    lp = torch.randn(2, 5)
    sig = SignalBatch(log_prob=lp, aux={"token_mask": torch.zeros(2, 5)})
    loss, m = algo.compute_signal_loss(sig, torch.ones(2), lp + 1.0)
    assert loss.item() == 0.0 and m.clip_fraction == 0.0


def test_clip_fraction_one_at_huge_ratio():
    algo = TokenGRPO(TokenGRPOConfig(eps_clip=0.2))
    sig = SignalBatch(log_prob=torch.full((2, 3), 5.0), aux={})
    _, m = algo.compute_signal_loss(sig, torch.ones(2), torch.zeros(2, 3))
    assert m.clip_fraction == 1.0


def test_k1_and_k3_estimators():
    lp = torch.full((1, 4), 0.5)
    ref = torch.zeros(1, 4)
    k1 = TokenGRPO(TokenGRPOConfig(init_kl_coef=1.0, kl_estimator="k1"))
    _, m1 = k1.compute_signal_loss(SignalBatch(log_prob=lp, ref_log_prob=ref), torch.zeros(1), lp)
    assert m1.kl_penalty == pytest.approx(0.5)
    k3 = TokenGRPO(TokenGRPOConfig(init_kl_coef=1.0, kl_estimator="k3"))
    _, m3 = k3.compute_signal_loss(SignalBatch(log_prob=lp, ref_log_prob=ref), torch.zeros(1), lp)
    assert m3.kl_penalty == pytest.approx(math.exp(0.5) * (0.5 - 1) + 1) and m3.kl_penalty >= 0


def test_kl_skipped_without_reference_and_errors():
    algo = TokenGRPO(TokenGRPOConfig(init_kl_coef=1.0))
    lp = torch.zeros(1, 3)
    _, m = algo.compute_signal_loss(SignalBatch(log_prob=lp), torch.zeros(1), lp)
    assert m.kl_penalty == 0.0
    with pytest.raises(ValueError, match="kl_estimator"):
        TokenGRPO(TokenGRPOConfig(kl_estimator="k9")).compute_signal_loss(
            SignalBatch(log_prob=lp), torch.zeros(1), lp)
    with pytest.raises(ValueError, match="shape mismatch"):
        algo.compute_signal_loss(SignalBatch(log_prob=lp), torch.zeros(1), torch.zeros(1, 4))
