"""Evaluators and the SDE step they are built on, against stub policies and a six-point schedule.

Re-expresses what the reference pins in ``tests/rollouts/test_evaluators.py``: SDE-step shapes, sde
versus cps, determinism, ``prev_sample`` pass-through; replay goes through ``model.replay_forward``;
a reference that *is* the policy runs inside ``disable_adapter()``, a distinct one is called
directly; token evaluators gather ``log_softmax`` and refuse a reference that would equal the
policy; the latent KL is zero for equal means and grows when the step scale enters.
"""

import contextlib
import types

import pytest
import torch

from visionrl_b200.algorithms.flow_matching import compute_kl_divergence, sde_step_with_logprob
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.evaluators.ar import ContinuousTokenLogProbEvaluator, TokenLogProbEvaluator
from visionrl_b200.rollouts.evaluators.diffusion import FlowMatchingEvaluator
from visionrl_b200.rollouts.evaluators.types import SignalRequest


class MockScheduler:
    def __init__(self):
        self.sigmas = torch.tensor([1.0, 0.8, 0.6, 0.4, 0.2, 0.0])
        self.timesteps = torch.tensor([1000.0, 800.0, 600.0, 400.0, 200.0])

    def index_for_timestep(self, t):
        return int(torch.argmin((self.timesteps - float(t)).abs()))


def _latents(b=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(b, 4, 6, 6, generator=g), torch.randn(b, 4, 6, 6, generator=g)


# ------------------------------------------------------------------------------- the SDE step
@pytest.mark.parametrize("sde_type", ["sde", "cps"])
def test_step_shapes_and_finite_values(sde_type):
    v, x = _latents()
    t = torch.full((3,), 600.0)
    res = sde_step_with_logprob(MockScheduler(), v, t, x, generator=torch.Generator().manual_seed(1),
                                noise_level=0.7, sde_type=sde_type, return_dt=True)
    assert res.prev_sample.shape == x.shape and res.prev_sample_mean.shape == x.shape
    assert res.log_prob.shape == (3,) and bool(torch.isfinite(res.log_prob).all())
    assert res.std_dev_t.shape[0] == 3 and res.dt is not None


def test_sde_and_cps_are_different_steps():
    v, x = _latents()
    t = torch.full((3,), 400.0)
    kw = dict(generator=None, deterministic=False, noise_level=0.7)
    a = sde_step_with_logprob(MockScheduler(), v, t, x, prev_sample=x * 0.9, sde_type="sde", **kw)
    b = sde_step_with_logprob(MockScheduler(), v, t, x, prev_sample=x * 0.9, sde_type="cps", **kw)
    assert not torch.allclose(a.prev_sample_mean, b.prev_sample_mean)
    assert not torch.allclose(a.log_prob, b.log_prob)
    assert bool((b.log_prob <= 0).all())           # cps scores with a negative mean square


def test_same_generator_seed_same_sample_and_prev_sample_is_passed_through():
    v, x = _latents()
    t = torch.full((3,), 800.0)
    runs = [sde_step_with_logprob(MockScheduler(), v, t, x, generator=torch.Generator().manual_seed(9),
                                  noise_level=0.7) for _ in range(2)]
    assert torch.equal(runs[0].prev_sample, runs[1].prev_sample)
    given = torch.randn_like(x)
    replay = sde_step_with_logprob(MockScheduler(), v, t, x, prev_sample=given, noise_level=0.7)
    assert replay.prev_sample is given or torch.equal(replay.prev_sample, given)
    # the replayed log-prob of the rollout's own sample equals the rollout log-prob
    again = sde_step_with_logprob(MockScheduler(), v, t, x, prev_sample=runs[0].prev_sample, noise_level=0.7)
    assert torch.allclose(again.log_prob, runs[0].log_prob, atol=1e-6)


def test_per_sample_timesteps_pick_per_sample_sigmas():
    v, x = _latents()
    mixed = torch.tensor([800.0, 400.0, 200.0])
    res = sde_step_with_logprob(MockScheduler(), v, mixed, x, prev_sample=x, noise_level=0.7)
    singles = [sde_step_with_logprob(MockScheduler(), v[i:i + 1], mixed[i:i + 1], x[i:i + 1],
                                     prev_sample=x[i:i + 1], noise_level=0.7).log_prob for i in range(3)]
    assert torch.allclose(res.log_prob, torch.cat(singles), atol=1e-6)


# ------------------------------------------------------------------------- flow-matching evaluator
class ReplayPolicy:
    """Counts replay calls and records whether the adapter was off during each."""

    def __init__(self, offset=0.0):
        self.offset = offset
        self.adapter_off = False
        self.calls = []

    def replay_forward(self, batch, timestep_idx):
        self.calls.append((timestep_idx, self.adapter_off))
        pred = batch.observations[:, timestep_idx] * 0.1 + self.offset
        return {"noise_pred": pred - (0.05 if self.adapter_off else 0.0)}

    @contextlib.contextmanager
    def disable_adapter(self):
        self.adapter_off = True
        try:
            yield
        finally:
            self.adapter_off = False


def _diffusion_batch(b=4, t=3):
    g = torch.Generator().manual_seed(2)
    obs = torch.randn(b, t, 4, 6, 6, generator=g)
    ts = torch.tensor([800.0, 600.0, 400.0]).expand(b, t).contiguous()
    return RolloutBatch(observations=obs, actions=obs + 0.05 * torch.randn(b, t, 4, 6, 6, generator=g),
                        rewards=torch.zeros(b), dones=torch.ones(b), group_ids=torch.zeros(b, dtype=torch.long),
                        extras={"timesteps": ts, "log_probs": torch.zeros(b, t)}, context={})


def test_replay_goes_through_the_policy_and_no_reference_unless_asked():
    policy, batch = ReplayPolicy(), _diffusion_batch()
    ev = FlowMatchingEvaluator(MockScheduler(), noise_level=0.7)
    sig = ev.evaluate(policy, batch, 1)
    assert policy.calls == [(1, False)]
    assert sig.log_prob.shape == (4,) and sig.ref_log_prob is None and sig.dist_family == "flow_matching"
    assert sig.prev_sample_mean.shape == batch.observations[:, 1].shape
    # a reference is computed only when the request asks for one
    ev.evaluate(policy, batch, 1, ref_model=policy)
    assert policy.calls == [(1, False), (1, False)]


def test_reference_that_is_the_policy_runs_with_the_adapter_off():
    policy, batch = ReplayPolicy(), _diffusion_batch()
    ev = FlowMatchingEvaluator(MockScheduler(), noise_level=0.7)
    sig = ev.evaluate(policy, batch, 2, ref_model=policy,
                      signal_request=SignalRequest(need_ref=True, need_kl_intermediates=True))
    assert [off for _, off in policy.calls] == [False, True]
    assert policy.adapter_off is False                         # restored afterwards
    assert sig.ref_log_prob is not None and not torch.allclose(sig.ref_log_prob, sig.log_prob)
    assert sig.ref_prev_sample_mean is not None and sig.dt is not None and sig.std_dev_t is not None
    assert not sig.ref_log_prob.requires_grad


def test_distinct_reference_model_is_called_directly():
    policy, ref, batch = ReplayPolicy(), ReplayPolicy(offset=0.3), _diffusion_batch()
    ev = FlowMatchingEvaluator(MockScheduler(), noise_level=0.7)
    sig = ev.evaluate(policy, batch, 0, ref_model=ref, signal_request=SignalRequest(need_ref=True))
    assert policy.calls == [(0, False)] and ref.calls == [(0, False)]
    assert not torch.allclose(sig.ref_prev_sample_mean, sig.prev_sample_mean)


def test_gradient_reaches_the_policy_output_only():
    class Learnable(ReplayPolicy):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.tensor(0.1))

        def replay_forward(self, batch, timestep_idx):
            return {"noise_pred": batch.observations[:, timestep_idx] * self.w}

    policy, batch = Learnable(), _diffusion_batch()
    sig = FlowMatchingEvaluator(MockScheduler(), noise_level=0.7).evaluate(
        policy, batch, 1, ref_model=policy, signal_request=SignalRequest(need_ref=True))
    sig.log_prob.sum().backward()
    assert policy.w.grad is not None and float(policy.w.grad.abs()) > 0


# --------------------------------------------------------------------------------- KL helper
def test_latent_kl_zero_for_equal_means_and_larger_with_small_dt():
    mean = torch.randn(3, 4, 6, 6)
    std = torch.full((3, 1, 1, 1), 0.5)
    assert torch.allclose(compute_kl_divergence(mean, mean, std), torch.zeros(3))
    other = mean + 0.2
    plain = compute_kl_divergence(mean, other, std)
    with_dt = compute_kl_divergence(mean, other, std, dt=torch.full((3, 1, 1, 1), 0.1))
    assert bool((with_dt > plain).all())
    assert torch.allclose(plain, torch.full((3,), 0.2 ** 2 / (2 * 0.25)), atol=1e-6)


# -------------------------------------------------------------------------------- token evaluators
class TokenPolicy:
    def __init__(self, vocab=11, adapters=True, bias=0.0):
        self.vocab, self.bias = vocab, bias
        self.has_adapters = adapters
        self.adapter_off = False
        self.calls = 0

    def replay_forward(self, batch, timestep_idx=0):
        self.calls += 1
        b, length = batch.actions.shape
        g = torch.Generator().manual_seed(4)
        logits = torch.randn(b, length, self.vocab, generator=g) + self.bias
        if self.adapter_off:
            logits = logits * 0.5
        return {"logits": logits.requires_grad_(True)}

    @contextlib.contextmanager
    def disable_adapter(self):
        self.adapter_off = True
        try:
            yield
        finally:
            self.adapter_off = False


def _token_batch(b=2, length=5, vocab=11, temperature=1.0):
    ids = torch.randint(0, vocab, (b, length), generator=torch.Generator().manual_seed(5))
    return RolloutBatch(observations=torch.zeros(b, 1, 3, dtype=torch.long), actions=ids,
                        rewards=torch.zeros(b), dones=torch.ones(b), group_ids=torch.zeros(b, dtype=torch.long),
                        extras={"token_mask": torch.ones(b, length), "log_probs": torch.zeros(b, 1, length)},
                        context={"temperature": temperature})


def test_token_evaluator_gathers_log_softmax_and_forwards_the_mask():
    policy, batch = TokenPolicy(), _token_batch()
    sig = TokenLogProbEvaluator().evaluate(policy, batch)
    logits = policy.replay_forward(batch)["logits"].detach()
    want = torch.log_softmax(logits.float(), dim=-1).gather(-1, batch.actions.unsqueeze(-1)).squeeze(-1)
    assert torch.allclose(sig.log_prob, want, atol=1e-6)
    assert sig.dist_family == "categorical" and "token_mask" in sig.aux and sig.ref_log_prob is None
    assert sig.log_prob.requires_grad


def test_token_evaluator_divides_by_the_recorded_temperature():
    policy = TokenPolicy()
    hot = TokenLogProbEvaluator().evaluate(policy, _token_batch(temperature=2.0)).log_prob
    logits = policy.replay_forward(_token_batch())["logits"].detach()
    want = torch.log_softmax(logits.float() / 2.0, dim=-1).gather(
        -1, _token_batch().actions.unsqueeze(-1)).squeeze(-1)
    assert torch.allclose(hot, want, atol=1e-6)


def test_token_reference_uses_adapter_off_or_a_distinct_model_and_never_the_policy_itself():
    batch = _token_batch()
    policy = TokenPolicy()
    sig = TokenLogProbEvaluator().evaluate(policy, batch, ref_model=policy,
                                           signal_request=SignalRequest(need_ref=True))
    assert policy.calls == 2 and not torch.allclose(sig.ref_log_prob, sig.log_prob)
    assert not sig.ref_log_prob.requires_grad
    other = TokenPolicy(bias=1.0)
    sig2 = TokenLogProbEvaluator().evaluate(policy, batch, ref_model=other,
                                            signal_request=SignalRequest(need_ref=True))
    assert other.calls == 1 and sig2.ref_log_prob is not None
    bare = TokenPolicy(adapters=False)
    with pytest.raises(RuntimeError, match="no adapter"):
        TokenLogProbEvaluator().evaluate(bare, batch, signal_request=SignalRequest(need_ref=True))


def test_continuous_token_evaluator_unwraps_replayed_log_probs():
    class FlowTokenPolicy:
        has_adapters = True

        def __init__(self):
            self.off = False

        def replay_forward(self, batch, timestep_idx=0):
            base = torch.arange(batch.actions.shape[0] * batch.actions.shape[1], dtype=torch.float32)
            return {"log_probs": base.view(batch.actions.shape[:2]) * (0.5 if self.off else 1.0)}

        @contextlib.contextmanager
        def disable_adapter(self):
            self.off = True
            try:
                yield
            finally:
                self.off = False

    b, length, dim = 2, 4, 3
    batch = RolloutBatch(observations=torch.zeros(b, 1, 3, dtype=torch.long), actions=torch.zeros(b, length, dim),
                         rewards=torch.zeros(b), dones=torch.ones(b), group_ids=torch.zeros(b, dtype=torch.long),
                         extras={"token_mask": torch.ones(b, length)}, context={})
    policy = FlowTokenPolicy()
    sig = ContinuousTokenLogProbEvaluator().evaluate(policy, batch, ref_model=policy,
                                                     signal_request=SignalRequest(need_ref=True))
    assert sig.log_prob.shape == (b, length)
    assert torch.allclose(sig.ref_log_prob, sig.log_prob * 0.5)
    assert "token_mask" in sig.aux
