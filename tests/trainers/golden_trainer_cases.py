"""Two trainer steps in three set-ups (clipped group loss; the same with the per-prompt statistics
tracker; the token-level loss with a frozen reference model and the k3 estimator) on a small MLP,
a collector that returns seeded rollouts and an evaluator that reads log-probabilities off the
model.  ``compute()`` returns every metric of every step, the order in which timesteps were
evaluated, the parameters after the four optimiser steps, the averaged parameters and the step
counters; ``tests/golden/trainer_outputs.pt`` holds what the reference's trainer, algorithms and
tracker give for exactly this."""

import asyncio
import inspect

import torch
from torch import nn
from vrl.algorithms.grpo import GRPO, GRPOConfig
from vrl.algorithms.grpo_token import TokenGRPO, TokenGRPOConfig
from vrl.algorithms.stat_tracking import PerPromptStatTracker
from vrl.rollouts.batch import RolloutBatch
from vrl.rollouts.evaluators import SignalBatch
from vrl.trainers.online import OnlineTrainer
from vrl.trainers.types import TrainerConfig
import vrl.trainers.types as T
import inspect
fields = set(inspect.signature(SignalBatch).parameters)
def sig(**kw): return SignalBatch(**{k: v for k, v in kw.items() if k in fields})

class Collector:
    def __init__(self, timesteps, token=False): self.t, self.token, self.calls = timesteps, token, 0
    async def collect(self, prompts, group_size, **kw):
        self.calls += 1
        g = torch.Generator().manual_seed(100 + self.calls)
        b = len(prompts) * group_size
        L = 5
        obs = torch.randn(b, 1, L, 3, generator=g) if self.token else torch.randn(b, self.t, 3, generator=g)
        rewards = torch.randn(b, generator=g)
        lp = torch.randn(b, 1, L, generator=g) * 0.1 if self.token else torch.randn(b, self.t, generator=g) * 0.1
        extras = {"log_probs": lp}
        if self.token:
            extras["token_mask"] = (torch.rand(b, L, generator=g) > 0.2).float()
        return RolloutBatch(observations=obs, actions=obs + 1, rewards=rewards, dones=torch.ones(b),
                            group_ids=torch.arange(len(prompts)).repeat_interleave(group_size), extras=extras, context={},
                            prompts=[p for p in prompts for _ in range(group_size)])

class Evaluator:
    def __init__(self, token=False): self.token = token; self.seen = []
    def evaluate(self, model, batch, timestep_idx, ref_model=None, signal_request=None):
        self.seen.append(int(timestep_idx))
        if self.token:
            x = batch.observations[:, timestep_idx]                  # [B, L, 3]
            lp = model(x).squeeze(-1) * 0.1
            ref = None
            if ref_model is not None:
                with torch.no_grad(): ref = ref_model(x).squeeze(-1) * 0.1
            return sig(log_prob=lp, ref_log_prob=ref, aux={"token_mask": batch.extras["token_mask"]}, dist_family="categorical")
        x = batch.observations[:, timestep_idx]
        return sig(log_prob=model(x).squeeze(-1) * 0.1, aux={}, dist_family="flow_matching")

def run(case):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(3, 4), nn.Tanh(), nn.Linear(4, 1))
    kw = dict(n=2, rollout_batch_size=4, bf16=False, timestep_fraction=0.5, ppo_epochs=2, max_norm=1.0)
    ema_cls = getattr(T, "EMAConfig")
    optim_cls = getattr(T, "OptimConfig", None)
    cfg = TrainerConfig(**kw, ema=ema_cls(enable=True, decay=0.9, update_interval=1))
    cfg.optim.lr = 1e-2
    token = case == "token"
    if token:
        algo = TokenGRPO(TokenGRPOConfig(eps_clip=0.2, init_kl_coef=0.05, kl_estimator="k3"))
        ref = nn.Sequential(nn.Linear(3, 4), nn.Tanh(), nn.Linear(4, 1))
        ref.load_state_dict(model.state_dict())
        for p in ref.parameters(): p.requires_grad_(False)
        cfg.timestep_fraction = 1.0
    else:
        algo, ref = GRPO(GRPOConfig(eps_clip=0.2, adv_clip_max=1.0)), None
    tracker = PerPromptStatTracker() if case == "tracker" else None
    col, ev = Collector(1 if token else 4, token), Evaluator(token)
    tr = OnlineTrainer(algo, col, ev, model, ref_model=ref, config=cfg, prompts=["a", "b", "c", "d"], device="cpu", stat_tracker=tracker)
    res = {}
    loop = asyncio.new_event_loop()
    for step in range(2):
        m = loop.run_until_complete(tr.step())
        for k in ("loss", "policy_loss", "kl_penalty", "reward_mean", "reward_std", "clip_fraction", "approx_kl", "advantage_mean",
                  "grad_norm", "adv_saturation", "adv_zero_rate", "group_size", "trained_prompt_num"):
            res[f"{case}/step{step}/{k}"] = torch.tensor(float(getattr(m, k)))
    res[f"{case}/seen"] = torch.tensor(ev.seen)
    for n, p in model.named_parameters(): res[f"{case}/param/{n}"] = p.detach().clone()
    res[f"{case}/state"] = torch.tensor([tr.state.step, tr.state.global_step])
    sd = tr.state_dict()
    res[f"{case}/state_keys"] = torch.tensor([float(len(k)) for k in sorted(sd)])
    ema = sd.get("ema")
    if ema is not None:
        vals = ema.get("ema_parameters") or ema.get("shadow_params") or []
        for i, v in enumerate(vals): res[f"{case}/ema/{i}"] = v.detach().clone().float()
    return res


def compute() -> dict:
    res = {}
    for case in ("plain", "tracker", "token"):
        res.update(run(case))
    return res
