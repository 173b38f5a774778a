"""SDE / CPS step: shapes, determinism, replay consistency, parity with the written formulas."""

import math

import pytest
import torch

from vrl.algorithms import sde_step_with_logprob
from vrl.algorithms.stat_tracking import PerPromptStatTracker


class MockScheduler:
    def __init__(self):
        self.sigmas = torch.tensor([1.0, 0.8, 0.6, 0.4, 0.2, 0.0])
        self.timesteps = self.sigmas[:-1] * 1000

    def index_for_timestep(self, t):
        return int(torch.argmin((self.timesteps - float(t)).abs()))


def _formula_sde(sched, v, t, x, prev, noise_level):
    i = sched.index_for_timestep(t[0])
    s, sn = sched.sigmas[i], sched.sigmas[i + 1]
    smax, smin = sched.sigmas[1], sched.sigmas[-1]
    dt = sn - s
    if noise_level != 1.0:
        std = torch.sqrt(s / (1 - (smax if s == 1 else s))) * noise_level
    else:
        std = smin + (smax - smin) * s
    mu = x * (1 + std**2 / (2 * s) * dt) + v * (1 + std**2 * (1 - s) / (2 * s)) * dt
    nu = std * torch.sqrt(-dt)
    lp = (-((prev - mu) ** 2) / (2 * nu**2) - torch.log(nu) - math.log(math.sqrt(2 * math.pi)))
    return mu, lp.mean(dim=tuple(range(1, x.ndim)))


@pytest.mark.parametrize("noise_level", [1.0, 0.7])
@pytest.mark.parametrize("step", [0, 2])
def test_sde_matches_written_formula(noise_level, step):
    torch.manual_seed(0)
    sched = MockScheduler()
    v, x, prev = (torch.randn(3, 4, 5, 5) for _ in range(3))
    t = sched.timesteps[step].expand(3)
    res = sde_step_with_logprob(sched, v, t, x, prev_sample=prev, noise_level=noise_level)
    mu, lp = _formula_sde(sched, v, t, x, prev, noise_level)
    assert torch.allclose(res.prev_sample_mean, mu, atol=1e-5)
    assert torch.allclose(res.log_prob, lp, rtol=1e-4, atol=1e-4)
    assert res.log_prob.shape == (3,) and res.dt is None


def test_cps_differs_from_sde_and_uses_negative_square():
    sched = MockScheduler()
    torch.manual_seed(1)
    v, x, prev = (torch.randn(2, 3, 4, 4) for _ in range(3))
    t = sched.timesteps[1].expand(2)
    a = sde_step_with_logprob(sched, v, t, x, prev_sample=prev, sde_type="sde")
    b = sde_step_with_logprob(sched, v, t, x, prev_sample=prev, sde_type="cps", noise_level=0.8)
    assert not torch.allclose(a.log_prob, b.log_prob)
    assert torch.allclose(b.log_prob, -((prev - b.prev_sample_mean) ** 2).mean(dim=(1, 2, 3)))


def test_generator_determinism_and_replay_roundtrip():
    sched = MockScheduler()
    v, x = torch.randn(2, 3, 4, 4), torch.randn(2, 3, 4, 4)
    t = sched.timesteps[0].expand(2)
    outs = [sde_step_with_logprob(sched, v, t, x, generator=torch.Generator().manual_seed(7),
                                  noise_level=0.7) for _ in range(2)]
    assert torch.equal(outs[0].prev_sample, outs[1].prev_sample)
    replay = sde_step_with_logprob(sched, v, t, x, prev_sample=outs[0].prev_sample,
                                   noise_level=0.7, return_dt=True)
    assert torch.equal(replay.log_prob, outs[0].log_prob)
    assert torch.allclose(replay.dt.flatten(), torch.full((2,), math.sqrt(0.2)))


def test_deterministic_step_and_argument_errors():
    sched = MockScheduler()
    v, x = torch.randn(2, 3), torch.randn(2, 3)
    t = sched.timesteps[2].expand(2)
    res = sde_step_with_logprob(sched, v, t, x, deterministic=True)
    assert torch.allclose(res.prev_sample, x + (0.4 - 0.6) * v, atol=1e-6)
    with pytest.raises(ValueError, match="both generator and prev_sample"):
        sde_step_with_logprob(sched, v, t, x, prev_sample=x, generator=torch.Generator())
    with pytest.raises(ValueError, match="sde_type"):
        sde_step_with_logprob(sched, v, t, x, sde_type="ode")


def test_gradient_flows_to_model_output():
    sched = MockScheduler()
    v = torch.randn(2, 3, 4, requires_grad=True)
    x, prev = torch.randn(2, 3, 4), torch.randn(2, 3, 4)
    res = sde_step_with_logprob(sched, v, sched.timesteps[1].expand(2), x, prev_sample=prev)
    res.log_prob.sum().backward()
    assert v.grad is not None and v.grad.abs().sum() > 0


def test_stat_tracker_grpo_and_history():
    tr = PerPromptStatTracker()
    adv = tr.update(["a", "a", "b", "b"], torch.tensor([1.0, 3.0, 2.0, 2.0]))
    assert adv[0] == pytest.approx(-1 / (1 + 1e-4)) and adv[2] == 0.0
    assert tr.get_stats() == (2.0, 2)
    tr.clear()
    assert tr.get_stats() == (0.0, 0) or tr.get_stats()[0] == 0.0
    assert tr.update(["a", "a"], [0.0, 1.0], type="dpo").tolist() == [-1.0, 1.0]
    assert tr.update(["c", "c"], [0.5, 0.7], type="sft").tolist() == [0.0, 1.0]
    with pytest.raises(ValueError):
        tr.update(["a"], [1.0], type="nope")
