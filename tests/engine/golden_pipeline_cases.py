"""A stub diffusion policy (one trainable scalar, deterministic arithmetic) driven through the real
rollout path: executor (micro-batching, seeds, SDE / CPS steps, the stochastic window, KL recording,
one shared starting latent) -> packer (rewards, KL-shaped rewards, extras, context) -> evaluator
(replayed log-probabilities, step means, the adapter-off reference and its KL inputs) for six
sampling set-ups.  ``compute()`` flattens everything that comes out into named tensors;
``tests/golden/rollout_pipeline_outputs.pt`` holds what the reference's executor base, packer and
evaluator give for the same stub."""

import asyncio
import contextlib
import random
from dataclasses import dataclass, field
from typing import Any

import torch

from vrl.engine.core.types import GenerationRequest
from vrl.engine.core.worker import GenerationIdFactory
from vrl.engine.diffusion.executor_base import DiffusionPipelineExecutorBase
from vrl.rollouts.evaluators.diffusion import FlowMatchingEvaluator
from vrl.rollouts.evaluators import SignalRequest
from vrl.rollouts.packers.base import RolloutPackContext
from vrl.rollouts.packers.diffusion import DiffusionRolloutPacker
T = 4
class Sched:
    def __init__(self):
        s = torch.linspace(1.0, 1.0 / 1000, T, dtype=torch.float64)
        s = 3.0 * s / (1 + 2.0 * s)
        self.timesteps = (s * 1000).float()
        self.sigmas = torch.cat([s, s.new_zeros(1)]).float()
    def index_for_timestep(self, t): return int(torch.argmin((self.timesteps - float(t)).abs()))
    def indices_for_timesteps(self, ts):
        ts = torch.as_tensor(ts, dtype=torch.float32).reshape(-1)
        return torch.argmin((ts[:, None] - self.timesteps[None]).abs(), dim=1)
    def set_timesteps(self, n, device=None): pass
@dataclass
class State:
    latents: torch.Tensor
    timesteps: torch.Tensor
    scheduler: Any
    prompt_embeds: torch.Tensor
    extra: dict = field(default_factory=dict)
class Policy(torch.nn.Module):
    device = torch.device("cpu")
    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.tensor(0.1))
        self.adapter = True
    def encode_prompt(self, prompt, negative_prompt=None, **kw):
        plist = [prompt] if isinstance(prompt, str) else list(prompt)
        return {"prompt_embeds": torch.stack([torch.full((3, 2), float(sum(ord(c) for c in p) % 7)) for p in plist])}
    def prepare_sampling(self, request, encoded, **kw):
        b = encoded["prompt_embeds"].shape[0]
        gen = torch.Generator().manual_seed(int(request.seed if request.seed is not None else 0))
        s = Sched()
        return State(torch.randn(b, 2, 4, 4, generator=gen), s.timesteps, s, encoded["prompt_embeds"], dict(kw))
    def _pred(self, x, emb):
        w = self.w if self.adapter else self.w.detach() * 0.5
        return w * x + emb.mean(dim=(1, 2)).view(-1, 1, 1, 1) * 0.01
    def forward_step(self, state, i):
        p = self._pred(state.latents, state.prompt_embeds)
        return {"noise_pred": p, "noise_pred_cond": p, "noise_pred_uncond": torch.zeros_like(p)}
    def decode_latents(self, latents): return latents[:, :1].repeat(1, 3, 1, 1).clamp(0, 1)
    def export_batch_context(self, state): return {"guidance_scale": 4.5, "model_family": "stub", "cfg": True}
    def export_training_extras(self, state): return {"prompt_embeds": state.prompt_embeds}
    def replay_forward(self, batch, j):
        p = self._pred(batch.observations[:, j].float(), batch.extras["prompt_embeds"])
        return {"noise_pred": p, "noise_pred_cond": p, "noise_pred_uncond": torch.zeros_like(p)}
    @contextlib.contextmanager
    def disable_adapter(self):
        self.adapter = False
        try: yield
        finally: self.adapter = True
class Ex(DiffusionPipelineExecutorBase):
    family, task = "sd3_5", "t2i"
    default_sample_batch_size = 4
    def __init__(self, policy): self.model = policy
def req(prompts, n, **s):
    base = {"num_steps": T, "guidance_scale": 4.5, "height": 32, "width": 32, "noise_level": 0.7, "sample_batch_size": 2, "seed": 5}
    base.update(s)
    return GenerationRequest(request_id="req", family="sd3_5", task="t2i", prompts=prompts, samples_per_prompt=n, sampling=base)
def flat(res, prefix, obj, depth=0):
    if torch.is_tensor(obj): res[prefix] = obj.detach().float().clone()
    elif isinstance(obj, dict):
        for k, v in sorted(obj.items(), key=lambda kv: str(kv[0])): flat(res, f"{prefix}.{k}", v, depth + 1)
    elif isinstance(obj, (int, float, bool)): res[prefix] = torch.tensor(float(obj))
    elif hasattr(obj, "__dataclass_fields__") and depth < 4:
        for k in obj.__dataclass_fields__: flat(res, f"{prefix}.{k}", getattr(obj, k), depth + 1)

def compute() -> dict:
    res = {}
    pol = Policy()
    ex = Ex(pol)
    cases = {"base": dict(), "kl": dict(return_kl=True), "cps": dict(sde_type="cps", noise_level=1.0), "window": dict(sde_window_size=2, sde_window_range=[0, 3]),
             "same": dict(same_latent=True), "nlow": dict(noise_level=0.3, sample_batch_size=3)}
    loop = asyncio.new_event_loop()
    for name, extra in cases.items():
        random.seed(11)
        r = req(["a cat", "b dog"], 3, **extra)
        o = ex.forward(r, GenerationIdFactory().build_sample_specs(r))
        flat(res, f"{name}/out", o.output)
        flat(res, f"{name}/traj", o.rollout_trajectory_data)
        flat(res, f"{name}/extra", o.extra if hasattr(o, "extra") else {})
        res[f"{name}/specs"] = torch.tensor([[s.prompt_index, s.sample_index] for s in o.sample_specs]).float()
        res[f"{name}/micro"] = torch.tensor(float(o.metrics.micro_batches))
        ctx = RolloutPackContext(metadata={}, device=torch.device("cpu"), kl_reward=0.01 if name == "kl" else 0.0, rescale_to_unit=False)
        batch = loop.run_until_complete(DiffusionRolloutPacker(error_prefix="Stub").pack(o, torch.arange(6.0), ctx))
        flat(res, f"{name}/batch.obs", batch.observations)
        flat(res, f"{name}/batch.act", batch.actions)
        flat(res, f"{name}/batch.rew", batch.rewards)
        flat(res, f"{name}/batch.gid", batch.group_ids.float())
        flat(res, f"{name}/batch.extras", batch.extras)
        flat(res, f"{name}/batch.ctx", batch.context)
        ev = FlowMatchingEvaluator(Sched(), noise_level=float(r.sampling["noise_level"]), sde_type=r.sampling.get("sde_type", "sde"))
        for j in range(T):
            sgn = ev.evaluate(pol, batch, j, ref_model=pol, signal_request=SignalRequest(need_ref=True, need_kl_intermediates=True))
            flat(res, f"{name}/sig{j}", sgn)
    return res
