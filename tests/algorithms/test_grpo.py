"""GRPO advantages, clipped loss and latent-space KL (closed-form expectations)."""

import math

import pytest
import torch

from vrl.algorithms import GRPO, GRPOConfig, compute_kl_divergence
from vrl.algorithms.grpo import group_normalized_advantages
from vrl.rollouts.evaluators.types import SignalBatch


def _loop_oracle(rewards, group_ids, eps, clip, global_std=False):
    adv = torch.zeros_like(rewards)
    for gid in torch.unique(group_ids):
        m = group_ids == gid
        r = rewards[m]
        if r.numel() <= 1:
            continue
        std = rewards.std() if global_std else r.std()
        adv[m] = ((r - r.mean()) / std.clamp(min=eps)).clamp(-clip, clip)
    return adv


def test_singleton_group_gets_zero_not_nan():
    g = GRPO(GRPOConfig())
    adv = g.compute_advantages_from_tensors(torch.tensor([3.0]), torch.tensor([0]))
    assert adv.tolist() == [0.0]


@pytest.mark.parametrize("global_std", [False, True])
def test_vectorised_advantages_match_loop(global_std):
    torch.manual_seed(0)
    rewards = torch.randn(23)
    groups = torch.randint(0, 5, (23,))
    groups[0] = 99  # singleton
    got = group_normalized_advantages(rewards, groups, 1e-8, 5.0, global_std)
    assert torch.allclose(got, _loop_oracle(rewards, groups, 1e-8, 5.0, global_std), atol=1e-6)


def test_constant_group_is_clipped_not_inf():
    g = GRPO(GRPOConfig(adv_clip_max=5.0))
    adv = g.compute_advantages_from_tensors(torch.tensor([1.0, 1.0, 1.0]), torch.tensor([0, 0, 0]))
    assert torch.isfinite(adv).all() and adv.abs().max() <= 5.0


def _signals(**kw):
    return SignalBatch(log_prob=torch.zeros(4), **kw)


def test_latent_kl_half_without_dt_and_fifty_with_dt():
    mu = torch.ones(4, 2, 2, 2)
    ref = torch.zeros(4, 2, 2, 2)
    std = torch.ones(4, 1, 1, 1)
    assert torch.allclose(compute_kl_divergence(mu, ref, std), torch.full((4,), 0.5))
    dt = torch.full((4, 1, 1, 1), 0.1)
    assert torch.allclose(compute_kl_divergence(mu, ref, std, dt=dt), torch.full((4,), 50.0))
    for use_dt, want in ((False, 0.5), (True, 50.0)):
        algo = GRPO(GRPOConfig(init_kl_coef=1.0, flow_kl_use_dt=use_dt))
        sig = _signals(ref_log_prob=torch.zeros(4), prev_sample_mean=mu, ref_prev_sample_mean=ref,
                       std_dev_t=std, dt=dt)
        _, m = algo.compute_signal_loss(sig, torch.zeros(4), torch.zeros(4))
        assert m.kl_penalty == pytest.approx(want, rel=1e-5)


def test_kl_requested_without_reference_raises():
    algo = GRPO(GRPOConfig(init_kl_coef=0.1))
    with pytest.raises(RuntimeError, match="ref_log_prob"):
        algo.compute_signal_loss(_signals(), torch.zeros(4), torch.zeros(4))


def test_logprob_kl_fallback_and_clip_metrics():
    algo = GRPO(GRPOConfig(init_kl_coef=1.0, eps_clip=0.1))
    lp = torch.tensor([0.5, 0.5, 0.0, 0.0], requires_grad=True)
    sig = SignalBatch(log_prob=lp, ref_log_prob=torch.zeros(4), dist_family="categorical")
    loss, m = algo.compute_signal_loss(sig, torch.ones(4), torch.zeros(4))
    assert m.kl_penalty == pytest.approx(0.25)
    assert m.clip_fraction == pytest.approx(0.5)
    assert m.approx_kl == pytest.approx(0.5 * 0.125)
    loss.backward()
    # clipped samples (ratio e^0.5 > 1.1 with positive advantage) carry no policy gradient
    assert lp.grad[0] == pytest.approx(0.25)
    assert algo._last_policy_loss_tensor is not None and algo._last_kl_term_tensor is not None


def test_device_metric_vector_without_sync():
    algo = GRPO(GRPOConfig())
    algo.sync_metrics = False
    _, m = algo.compute_signal_loss(_signals(), torch.ones(4), torch.zeros(4))
    assert m.loss == 0.0 and algo.last_metric_tensor.shape == (5,)
