"""DPM-Solver++(2M) and UniPC flow solvers against closed forms and a fine Euler reference."""

import pytest
import torch

from visionrl_b200.models.nn.flow_solvers import (
    FlowDPMSolverMultistepScheduler, FlowUniPCMultistepScheduler, get_sampling_sigmas,
    retrieve_timesteps,
)

SOLVERS = [FlowDPMSolverMultistepScheduler, FlowUniPCMultistepScheduler]


def _sample(scheduler, velocity, x, steps, shift=3.0):
    scheduler.set_timesteps(steps, shift=shift)
    for i, t in enumerate(scheduler.timesteps):
        x = scheduler.step(velocity(x, float(scheduler.sigmas[i])), t, x)
    return x


def _euler(velocity, x, steps, shift=3.0):
    sig = torch.cat([get_sampling_sigmas(steps, shift), torch.zeros(1)]).tolist()
    for i in range(steps):
        x = x + (sig[i + 1] - sig[i]) * velocity(x, sig[i])
    return x


@pytest.mark.parametrize("solver", SOLVERS)
def test_constant_data_prediction_is_hit_exactly(solver):
    """With v = (x - x0) / sigma the data prediction is x0 at every step: any consistent solver
    must return exactly x0, whatever the step count."""
    torch.manual_seed(0)
    x0, noise = torch.randn(3, 5), torch.randn(3, 5)
    velocity = lambda x, s: (x - x0) / s  # noqa: E731
    for steps in (1, 2, 7):
        out = _sample(solver(), velocity, noise.clone(), steps)
        assert torch.allclose(out, x0, atol=1e-5)


def _gaussian_velocity(mu, std):
    """Exact marginal velocity field when the data are N(mu, std^2) and the noise is N(0, 1)."""
    def velocity(x, s):
        var = (1 - s) ** 2 * std ** 2 + s ** 2
        x0_hat = mu + (1 - s) * std ** 2 / var * (x - (1 - s) * mu)
        return (x - x0_hat) / s
    return velocity


@pytest.mark.parametrize("solver", SOLVERS)
def test_second_order_beats_euler_on_gaussian_data(solver):
    """For Gaussian data the probability-flow ODE has the closed-form end point mu + std * x(1).
    With the same number of model calls the multistep solvers land much closer to it than Euler,
    and their error falls faster than linearly in the step size."""
    torch.manual_seed(1)
    mu, std = 1.0, 0.5
    x1 = torch.randn(4, 6)
    exact = mu + std * x1
    velocity = _gaussian_velocity(mu, std)
    err_euler = (_euler(velocity, x1.clone(), 20) - exact).abs().max().item()
    err_20 = (_sample(solver(), velocity, x1.clone(), 20) - exact).abs().max().item()
    err_40 = (_sample(solver(), velocity, x1.clone(), 40) - exact).abs().max().item()
    assert err_20 < 0.35 * err_euler, (err_20, err_euler)
    assert err_40 < 0.4 * err_20, (err_40, err_20)          # better than first order


def test_grid_and_interface():
    sig = get_sampling_sigmas(10, shift=5.0)
    assert sig.shape == (10,) and float(sig[0]) == pytest.approx(1.0) and bool((sig[1:] < sig[:-1]).all())
    assert float(sig[-1]) == pytest.approx(5.0 * 0.1 / (1 + 4.0 * 0.1))
    sched = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1.0)
    ts, n = retrieve_timesteps(sched, sigmas=sig)
    assert n == 10 and torch.allclose(ts, sig * 1000)
    assert sched.sigmas.shape == (11,) and float(sched.sigmas[-1]) == 0.0
    assert sched.index_for_timestep(float(ts[3])) == 3
    with pytest.raises(ValueError):
        sched.set_timesteps(sigmas=[0.5, 0.7])
    x = torch.zeros(2, 2)
    for t in ts:
        x = sched.step(torch.zeros(2, 2), t, x)
    with pytest.raises(RuntimeError):
        sched.step(torch.zeros(2, 2), ts[-1], x)
    with pytest.raises(ValueError):
        FlowDPMSolverMultistepScheduler(solver_order=3)
