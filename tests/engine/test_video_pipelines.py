"""Wan 2.1 and Cosmos executors over tiny random-init networks on CPU: 5-D latents, batched or
sequential CFG, chunk gathering, replay equality (reference expectations:
``tests/engine/generation/test_pipeline_wan_2_1.py``, ``test_pipeline_cosmos.py``)."""

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.gather import DiffusionChunkGatherer
from visionrl_b200.engine.microbatching import MicroBatchPlan

STEPS = 3
TINY_WAN = ["model.random_init=true", "model.use_lora=false", "model.dtype=float32",
            "model.torch_compile.enable=false", "model.arch.num_layers=2", "model.arch.hidden_size=64",
            "model.arch.num_heads=2", "model.arch.ffn_dim=128", "model.arch.in_channels=4",
            "model.arch.text_dim=32", "model.arch.freq_dim=32", f"sampling.num_steps={STEPS}",
            "sampling.width=32", "sampling.height=32", "sampling.num_frames=5",
            "sampling.max_sequence_length=8", "distributed.rollout.gpus_per_worker=0"]


def _request(family, task, prompts, n, **extra):
    sampling = {"num_steps": STEPS, "guidance_scale": 4.0, "height": 32, "width": 32, "num_frames": 5,
                "max_sequence_length": 8, "noise_level": 0.7, "sde_type": "sde", "sample_batch_size": 2,
                "seed": 3}
    sampling.update(extra)
    return GenerationRequest(request_id="req", family=family, task=task, prompts=prompts,
                             samples_per_prompt=n, sampling=sampling)


@pytest.fixture(scope="module")
def wan():
    from visionrl_b200.models.families.wan_2_1.builder import build_wan_2_1_runtime_bundle_from_cfg
    from visionrl_b200.models.families.wan_2_1.executor import Wan_2_1PipelineExecutor

    cfg = load_config("experiment/wan_2_1_1_3b_grpo", overrides=TINY_WAN)
    bundle = build_wan_2_1_runtime_bundle_from_cfg(cfg, "cpu", torch.float32)
    return bundle, Wan_2_1PipelineExecutor(bundle.policy, sample_batch_size=2)


def test_wan_rollout_has_video_latents_and_reproduces(wan):
    bundle, ex = wan
    req = _request("wan_2_1", "t2v", ["a", "b"], 3)
    specs = GenerationIdFactory().build_sample_specs(req)
    out = ex.forward(req, specs)
    lat = out.rollout_trajectory_data.dit_trajectory.latents
    assert lat.ndim == 6 and lat.shape[:3] == (6, STEPS, 4)              # [B, T, C, F, h, w]
    assert out.rollout_trajectory_data.rollout_log_probs.shape == (6, STEPS)
    assert out.output.ndim == 5 and out.output.shape[:2] == (6, 3)        # [B, 3, F, H, W]
    assert out.metrics.micro_batches == 4                                 # per prompt: 2 + 1
    again = ex.forward(req, specs)
    assert torch.equal(lat, again.rollout_trajectory_data.dit_trajectory.latents)


def test_wan_chunks_gather_to_the_same_batch_as_forward(wan):
    _, ex = wan
    req = _request("wan_2_1", "t2v", ["a"], 3)
    specs = GenerationIdFactory().build_sample_specs(req)
    whole = ex.forward(req, specs)
    chunks = [ex.forward_chunk(req, MicroBatchPlan(prompt_index=0, prompt="a", sample_start=s, sample_count=c))
              for s, c in ((0, 2), (2, 1))]        # plan order: the gatherer concatenates as given
    gathered = DiffusionChunkGatherer(model_family="wan_2_1").gather_chunks(req, specs, chunks)
    assert torch.equal(gathered.rollout_trajectory_data.rollout_log_probs,
                       whole.rollout_trajectory_data.rollout_log_probs)


def test_wan_replay_reproduces_rollout_log_probs(wan):
    import asyncio

    from visionrl_b200.rollouts.evaluators.diffusion import FlowMatchingEvaluator
    from visionrl_b200.rollouts.packers.base import RolloutPackContext
    from visionrl_b200.rollouts.packers.diffusion import DiffusionRolloutPacker

    bundle, ex = wan
    req = _request("wan_2_1", "t2v", ["a"], 2)
    out = ex.forward(req, GenerationIdFactory().build_sample_specs(req))
    ctx = RolloutPackContext(metadata={}, device=torch.device("cpu"), kl_reward=0.0, rescale_to_unit=False)
    batch = asyncio.new_event_loop().run_until_complete(
        DiffusionRolloutPacker(error_prefix="Wan").pack(out, torch.zeros(2), ctx))
    ev = FlowMatchingEvaluator(bundle.scheduler, noise_level=0.7, sde_type="sde")
    for j in range(STEPS):
        sig = ev.evaluate(bundle.policy, batch, j)
        assert torch.allclose(sig.log_prob, batch.extras["log_probs"][:, j], atol=1e-5)


def test_wan_official_policy_samples_with_both_flow_solvers(wan):
    """The two-expert variant generates with UniPC and DPM-Solver++; both are deterministic for a
    seed, agree with each other far better than with a first-order run of the same length, and
    switch to the low-noise expert below the boundary timestep."""
    from visionrl_b200.models.diffusion import VideoGenerationRequest
    from visionrl_b200.models.families.wan_2_1.official_policy import WanT2VOfficialPolicy

    base = wan[0].policy
    policy = WanT2VOfficialPolicy.__new__(WanT2VOfficialPolicy)
    policy.__dict__.update(base.__dict__)
    policy.boundary = 0.5
    object.__setattr__(policy, "_low_noise", None)
    policy._prompt_cache = {}
    policy.attach_low_noise_expert()
    used = []
    original = policy._expert
    policy._expert = lambda t: used.append(float(t.flatten()[0])) or original(t)

    def run(solver, steps):
        req = VideoGenerationRequest(prompt="a red fox", num_steps=steps, guidance_scale=3.0, height=32,
                                     width=32, frame_count=5, seed=11, sample_solver=solver, shift=3.0,
                                     extra={"max_sequence_length": 8})
        return policy.sample(req, decode=False)

    uni, dpm = run("unipc", 8), run("dpmpp", 8)
    assert uni.shape == dpm.shape and uni.ndim == 5 and bool(torch.isfinite(uni).all())
    assert torch.equal(uni, run("unipc", 8))
    fine = run("dpmpp", 64)
    assert (uni - fine).abs().mean() < 0.2 * fine.abs().mean()
    assert (dpm - fine).abs().mean() < 0.2 * fine.abs().mean()
    assert max(used) >= 500.0 > min(used)                      # both experts were consulted
    assert len(policy._prompt_cache) == 1                      # one prompt, encoded once


def test_official_wan_variant_is_selectable_from_the_config_and_rolls_out():
    """``model.backend: official`` builds the two-expert variant: the second expert is a different
    network, the boundary comes from the config, the executor drives it like any other policy, and
    asking it for adapters is refused (it is rollout-only)."""
    from visionrl_b200.models.families.wan_2_1.builder import build_wan_2_1_runtime_bundle_from_cfg
    from visionrl_b200.models.families.wan_2_1.executor import Wan_2_1PipelineExecutor
    from visionrl_b200.models.families.wan_2_1.official_policy import WanT2VOfficialPolicy

    cfg = load_config("experiment/wan_2_1_1_3b_grpo",
                      overrides=TINY_WAN + ["model.backend=official", "+model.arch.boundary=0.5"])
    bundle = build_wan_2_1_runtime_bundle_from_cfg(cfg, "cpu", torch.float32)
    policy = bundle.policy
    assert isinstance(policy, WanT2VOfficialPolicy) and bundle.backend_kind == "official"
    assert policy.boundary == 0.5 and policy._low_noise is not None
    high = dict(policy.transformer.named_parameters())
    low = dict(policy._low_noise.named_parameters())
    assert any(not torch.equal(high[k], low[k]) for k in high) and not any(p.requires_grad for p in low.values())
    req = _request("wan_2_1", "t2v", ["a"], 2)
    out = Wan_2_1PipelineExecutor(policy, sample_batch_size=2).forward(
        req, GenerationIdFactory().build_sample_specs(req))
    assert out.error is None and out.rollout_trajectory_data.rollout_log_probs.shape == (2, STEPS)
    with pytest.raises(NotImplementedError):
        build_wan_2_1_runtime_bundle_from_cfg(
            load_config("experiment/wan_2_1_1_3b_grpo", overrides=[o for o in TINY_WAN if "use_lora" not in o]
                        + ["model.backend=official"]), "cpu", torch.float32)
    with pytest.raises(NotImplementedError, match="no adapter for backend"):
        build_wan_2_1_runtime_bundle_from_cfg(
            load_config("experiment/wan_2_1_1_3b_grpo", overrides=TINY_WAN + ["model.backend=vendor"]),
            "cpu", torch.float32)
