"""The diffusion executor base against a stub policy that counts what is asked of it.

Re-expresses the executor expectations of the reference's pipeline tests
(``tests/engine/generation/test_pipeline_sd3_5.py:266-418`` and the Wan / Cosmos analogues) without a
network: how many times prompts are encoded and the model is called, the shapes and the prompt-major
order of what comes back, seeds, the SDE window, KL recording, spec parsing and its errors, and
the out-of-memory bisection seen from the executor.
"""

from dataclasses import dataclass, field
from typing import Any

import pytest
import torch

from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.diffusion.executor_base import DiffusionPipelineExecutorBase
from visionrl_b200.engine.microbatching import MicroBatchPlan

T = 4


class _StubScheduler:
    def __init__(self):
        self.sigmas = torch.linspace(1.0, 0.0, T + 1)
        self.timesteps = self.sigmas[:-1] * 1000

    def index_for_timestep(self, t):
        return int(torch.argmin((self.timesteps - float(t)).abs()))

    def indices_for_timesteps(self, ts):
        ts = torch.as_tensor(ts, dtype=torch.float32).reshape(-1)
        return torch.argmin((ts[:, None] - self.timesteps[None]).abs(), dim=1)


@dataclass
class _State:
    latents: torch.Tensor
    timesteps: torch.Tensor
    scheduler: Any
    prompt_embeds: torch.Tensor
    extra: dict = field(default_factory=dict)


class _StubPolicy:
    device = torch.device("cpu")

    def __init__(self, oom_above: int | None = None):
        self.encoded, self.forward_calls, self.prepare_batches, self.decoded = [], 0, [], 0
        self.oom_above = oom_above

    def encode_prompt(self, prompt, negative_prompt=None, **kwargs):
        self.encoded.append(prompt)
        value = float(sum(ord(c) for c in prompt) % 7)
        return {"prompt_embeds": torch.full((1, 3, 2), value)}

    def prepare_sampling(self, request, encoded, **kwargs):
        b = encoded["prompt_embeds"].shape[0]
        if self.oom_above is not None and b > self.oom_above:
            raise RuntimeError("CUDA out of memory. Tried to allocate 1.00 GiB")
        self.prepare_batches.append(b)
        gen = torch.Generator().manual_seed(int(request.seed if request.seed is not None else 0))
        sched = _StubScheduler()
        return _State(torch.randn(b, 2, 4, 4, generator=gen), sched.timesteps, sched,
                      encoded["prompt_embeds"], dict(kwargs))

    def forward_step(self, state, i):
        self.forward_calls += 1
        pred = 0.1 * state.latents + state.prompt_embeds.mean(dim=(1, 2)).view(-1, 1, 1, 1) * 0.01
        return {"noise_pred": pred, "noise_pred_cond": pred, "noise_pred_uncond": torch.zeros_like(pred)}

    def decode_latents(self, latents):
        self.decoded += 1
        return latents[:, :1].repeat(1, 3, 1, 1).clamp(0, 1)

    def export_batch_context(self, state):
        return {"guidance_scale": 4.5, "model_family": "stub"}

    def export_training_extras(self, state):
        return {"prompt_embeds": state.prompt_embeds}


class _StubExecutor(DiffusionPipelineExecutorBase):
    family, task = "sd3_5", "t2i"
    default_sample_batch_size = 4

    def __init__(self, policy):
        self.model = policy


def _request(prompts, n, **sampling):
    base = {"num_steps": T, "guidance_scale": 4.5, "height": 32, "width": 32, "noise_level": 0.7,
            "sample_batch_size": 4, "seed": 5}
    base.update(sampling)
    return GenerationRequest(request_id="req", family="sd3_5", task="t2i", prompts=prompts,
                             samples_per_prompt=n, sampling=base)


def _run(executor, request):
    return executor.forward(request, GenerationIdFactory().build_sample_specs(request))


def test_two_prompts_four_samples_give_eight_rows_in_prompt_major_order():
    policy = _StubPolicy()
    out = _run(_StubExecutor(policy), _request(["alpha", "beta"], 4))
    data = out.rollout_trajectory_data
    assert data.rollout_log_probs.shape == (8, T)
    assert data.dit_trajectory.latents.shape == (8, T, 2, 4, 4)
    assert data.dit_trajectory.timesteps.shape == (8, T)
    assert data.denoising_env.extra["kl"].shape == (8, T)
    assert out.output.shape == (8, 3, 4, 4)
    assert [s.prompt_index for s in out.sample_specs] == [0] * 4 + [1] * 4
    assert policy.encoded == ["alpha", "beta"]                       # once per prompt
    embeds = data.denoising_env.extra["training_extras"]["prompt_embeds"]
    assert torch.equal(embeds[:4], embeds[:1].expand(4, -1, -1)) and not torch.equal(embeds[0], embeds[4])
    assert out.metrics.num_samples == 8 and out.metrics.num_steps == T and out.metrics.micro_batches == 2


def test_twelve_samples_in_batches_of_four_make_three_chunks_and_three_t_forwards():
    policy = _StubPolicy()
    out = _run(_StubExecutor(policy), _request(["alpha"], 12))
    assert policy.prepare_batches == [4, 4, 4] and policy.forward_calls == 3 * T
    assert policy.encoded == ["alpha"] and out.metrics.micro_batches == 3
    assert out.rollout_trajectory_data.rollout_log_probs.shape == (12, T)


def test_same_seed_same_bits_and_chunks_use_their_own_seed_offsets():
    a = _run(_StubExecutor(_StubPolicy()), _request(["alpha"], 8))
    b = _run(_StubExecutor(_StubPolicy()), _request(["alpha"], 8))
    la, lb = (o.rollout_trajectory_data.dit_trajectory.latents for o in (a, b))
    assert torch.equal(la, lb)
    assert torch.equal(a.rollout_trajectory_data.rollout_log_probs, b.rollout_trajectory_data.rollout_log_probs)
    other = _run(_StubExecutor(_StubPolicy()), _request(["alpha"], 8, seed=6))
    assert not torch.equal(la, other.rollout_trajectory_data.dit_trajectory.latents)


def test_kl_is_abs_log_prob_only_when_asked_for():
    plain = _run(_StubExecutor(_StubPolicy()), _request(["a"], 4))
    assert float(plain.rollout_trajectory_data.denoising_env.extra["kl"].abs().max()) == 0.0
    with_kl = _run(_StubExecutor(_StubPolicy()), _request(["a"], 4, return_kl=True))
    data = with_kl.rollout_trajectory_data
    assert torch.equal(data.denoising_env.extra["kl"], data.rollout_log_probs.abs())


def test_same_latent_without_a_seed_is_refused():
    with pytest.raises(ValueError, match="same_latent"):
        _run(_StubExecutor(_StubPolicy()), _request(["a"], 2, seed=None, same_latent=True))


def test_steps_outside_the_sde_window_are_deterministic():
    """With a one-step window, all other steps are x + dt * v: two different seeds for the noise
    generator differ only from the window step onwards."""
    ex = _StubExecutor(_StubPolicy())
    req = _request(["a"], 2, sde_window_size=1, sde_window_range=(2, 3))
    spec = ex.parse_spec(req)
    assert spec.sde.sde_window_size == 1 and spec.sde.sde_window_range == (2, 3)
    out = _run(ex, req)
    lat = out.rollout_trajectory_data.dit_trajectory.latents
    act = out.rollout_trajectory_data.denoising_env.extra["actions"]
    sched = _StubScheduler()
    for i in (0, 1, 3):
        dt = float(sched.sigmas[i + 1] - sched.sigmas[i])
        x = lat[:, i]
        v = 0.1 * x + out.rollout_trajectory_data.denoising_env.extra["training_extras"]["prompt_embeds"] \
            .mean(dim=(1, 2)).view(-1, 1, 1, 1) * 0.01
        assert torch.allclose(act[:, i], x + dt * v, atol=1e-5)
    dt2 = float(sched.sigmas[3] - sched.sigmas[2])
    assert not torch.allclose(act[:, 2], lat[:, 2] + dt2 * (0.1 * lat[:, 2]), atol=1e-4)


def test_spec_parsing_defaults_and_errors():
    ex = _StubExecutor(_StubPolicy())
    spec = ex.parse_spec(_request(["a"], 1, frame_count=9, fps=8))
    assert spec.base.num_frames == 9 and spec.base.fps == 8 and spec.base.sample_batch_size == 4
    assert spec.base.max_sequence_length == 512 and spec.sde.sde_type == "sde"
    assert spec.sde.sde_window_range == (0, T) and spec.sde.noise_level == 0.7
    with pytest.raises(ValueError, match="sde_type"):
        ex.parse_spec(_request(["a"], 1, sde_type="ode"))
    with pytest.raises(ValueError, match="sde_window_range"):
        ex.parse_spec(_request(["a"], 1, sde_window_range=5))
    with pytest.raises(KeyError):
        bad = _request(["a"], 1)
        del bad.sampling["num_steps"]
        ex.parse_spec(bad)
    video = ex.build_video_request("a", spec)
    assert video.frame_count == 9 and video.fps == 8 and video.extra == {"max_sequence_length": 512}


def test_out_of_memory_chunks_are_bisected_and_rows_stay_in_order():
    policy = _StubPolicy(oom_above=2)
    out = _run(_StubExecutor(policy), _request(["alpha", "beta"], 4))
    assert policy.prepare_batches == [2, 2, 2, 2]                    # 4 -> (2, 2) for each prompt
    assert [s.sample_index for s in out.sample_specs] == [0, 1, 2, 3, 0, 1, 2, 3]
    whole = _run(_StubExecutor(_StubPolicy()), _request(["alpha", "beta"], 4, sample_batch_size=2))
    assert torch.equal(out.rollout_trajectory_data.dit_trajectory.latents,
                       whole.rollout_trajectory_data.dit_trajectory.latents)


def test_single_chunk_entry_point_matches_forward_and_coverage_is_checked():
    ex = _StubExecutor(_StubPolicy())
    req = _request(["alpha"], 4)
    specs = GenerationIdFactory().build_sample_specs(req)
    chunks = [ex.forward_chunk(req, MicroBatchPlan(0, "alpha", 0, 2)),
              ex.forward_chunk(req, MicroBatchPlan(0, "alpha", 2, 2))]
    gathered = ex.gather_chunks(req, specs, chunks)
    assert gathered.rollout_trajectory_data.rollout_log_probs.shape == (4, T)
    with pytest.raises(ValueError, match="misaligned"):
        ex.gather_chunks(req, specs, chunks[:1])
