"""The variance-preserving forward process behind the ``epsilon`` / ``v_prediction`` targets of
the preference trainer, against the closed forms, and the trainer's use of it."""

import math

import pytest
import torch

from visionrl_b200.models.nn.scheduler import DDPMNoiseScheduler
from visionrl_b200.trainers.offline_dpo import OfflineDPOTrainer, OfflineDPOTrainerConfig


def test_schedule_is_monotone_and_spans_signal_to_noise():
    s = DDPMNoiseScheduler()
    a = s.alphas_cumprod
    assert a.shape == (1000,) and bool((a[1:] < a[:-1]).all())
    assert float(a[0]) == pytest.approx(1 - 0.00085, abs=1e-6) and float(a[-1]) < 0.01
    assert s.config.num_train_timesteps == 1000 and s.timesteps.tolist()[:2] == [999, 998]
    s.set_timesteps(10)
    assert s.timesteps.tolist() == [900, 800, 700, 600, 500, 400, 300, 200, 100, 0]
    with pytest.raises(ValueError):
        s.set_timesteps(0)


def test_noising_and_velocity_match_the_closed_forms_and_invert():
    s = DDPMNoiseScheduler()
    x0, eps = torch.randn(3, 4, 5, 5), torch.randn(3, 4, 5, 5)
    t = torch.tensor([0, 500, 999])
    a = s.alphas_cumprod[t].view(3, 1, 1, 1)
    xt, v = s.add_noise(x0, eps, t), s.get_velocity(x0, eps, t)
    assert torch.allclose(xt, a.sqrt() * x0 + (1 - a).sqrt() * eps, atol=1e-6)
    assert torch.allclose(v, a.sqrt() * eps - (1 - a).sqrt() * x0, atol=1e-6)
    # (x_t, v) is a rotation of (x_0, eps): both can be recovered
    assert torch.allclose(a.sqrt() * xt - (1 - a).sqrt() * v, x0, atol=1e-5)
    assert torch.allclose((1 - a).sqrt() * xt + a.sqrt() * v, eps, atol=1e-5)
    with pytest.raises(ValueError, match="out of range"):
        s.add_noise(x0, eps, torch.tensor([0, 1, 1000]))


class _Batch:
    captions = ["a", "b"]

    def __init__(self):
        self.latents = torch.randn(4, 4, 6, 6)

    def latents_winner_then_loser(self):
        return self.latents


@pytest.mark.parametrize("kind", ["epsilon", "v_prediction"])
def test_preference_trainer_steps_on_both_targets(kind):
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = torch.nn.Conv2d(4, 4, 3, padding=1)

        def forward(self, x):
            return self.conv(x)

    model, ref = Net(), Net()
    ref.load_state_dict(model.state_dict())
    seen = []

    def forward_fn(net, noisy, timesteps, ctx, extra=None):
        seen.append(timesteps.clone())
        return net(noisy)

    sched = DDPMNoiseScheduler(prediction_type=kind)
    trainer = OfflineDPOTrainer(model, ref, forward_fn, sched, lambda px: px, lambda caps: torch.zeros(len(caps), 1),
                                OfflineDPOTrainerConfig(prediction_type=kind, lr=1e-3, mixed_precision="no"),
                                device="cpu")
    first = trainer.step(_Batch())
    assert first.loss == pytest.approx(math.log(2.0), abs=1e-6) and first.grad_norm > 0
    # winner and loser of a pair share the timestep, which is an integer step of the schedule
    t = seen[0]
    assert t.dtype == torch.long and torch.equal(t[:2], t[2:]) and 0 <= int(t.min()) and int(t.max()) < 1000
    second = trainer.step(_Batch())
    assert math.isfinite(second.loss) and trainer.global_step == 2
