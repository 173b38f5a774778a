"""Three steps of the preference trainer in four set-ups (plain, with the winner-MSE term, with
two-step gradient accumulation, with Adafactor) on a small convolution, a frozen copy as reference
and seeded preference pairs.  The schedule's entry ``i`` has the timestep value ``i``, so "the i-th
entry" and "the timestep i" name the same thing and the order of the random draws is all that
decides the numbers.  ``compute()`` returns every metric, the timesteps the model was called with,
the weights and the step counter; ``tests/golden/preference_trainer_outputs.pt`` holds what the
reference's trainer gives."""

import types

import torch
from torch import nn
from vrl.trainers.offline_dpo import OfflineDPOTrainer, OfflineDPOTrainerConfig
class Sched:
    def __init__(self, n=50):
        # entry i has timestep value i, so "the i-th entry" and "the timestep i" are the same thing
        s = torch.linspace(0.02, 0.98, n, dtype=torch.float64)
        self.timesteps = torch.arange(n).float()
        self.sigmas = torch.cat([s, s.new_ones(1)]).float()
        self.config = types.SimpleNamespace(num_train_timesteps=1000)
    def scale_noise(self, sample, timestep, noise):
        idx = torch.argmin((timestep.float()[:, None] - self.timesteps[None]).abs(), dim=1)
        sig = self.sigmas[idx].view(-1, *([1] * (sample.ndim - 1)))
        return (1 - sig) * sample + sig * noise
class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.c = nn.Conv2d(4, 4, 3, padding=1)
    def forward(self, x): return self.c(x)
class Batch:
    captions = ["a", "b"]
    def __init__(self, seed):
        g = torch.Generator().manual_seed(seed)
        self.pixel_values = torch.randn(2, 8, 6, 6, generator=g)
    def stacked_winner_then_loser(self):
        w, l = self.pixel_values.chunk(2, dim=1)
        return torch.cat([w, l], dim=0)


def compute() -> dict:
    res = {}
    for case, kw in {"plain": {}, "sft": {"sft_weight": 0.5}, "accum": {"gradient_accumulation_steps": 2}, "adafactor": {"use_adafactor": True}}.items():
        torch.manual_seed(0)
        model, ref = Net(), Net()
        ref.load_state_dict(model.state_dict())
        with torch.no_grad(): model.c.weight.add_(0.01)
        seen = []
        def fwd(net, noisy, ts, ctx, extra=None):
            seen.append(ts.detach().float().clone())
            return net(noisy)
        tr = OfflineDPOTrainer(model, ref, fwd, Sched(), lambda px: px, lambda caps: torch.zeros(len(caps), 1),
                               OfflineDPOTrainerConfig(prediction_type="flow_matching", lr=1e-3, mixed_precision="no",
                                                       beta=50.0, **kw), device="cpu")
        torch.manual_seed(42)
        for step in range(3):
            m = tr.step(Batch(step))
            for k in ("loss", "raw_model_loss", "raw_ref_loss", "model_diff", "ref_diff", "implicit_acc", "sft_loss", "grad_norm"):
                res[f"{case}/step{step}/{k}"] = torch.tensor(float(getattr(m, k)))
        res[f"{case}/timesteps"] = torch.stack(seen)
        res[f"{case}/weight"] = model.c.weight.detach().clone()
        res[f"{case}/global_step"] = torch.tensor(float(tr.global_step))
    return res
