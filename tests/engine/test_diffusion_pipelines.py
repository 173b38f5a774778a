"""Diffusion executors over the tiny native policies (reference expectations:
``tests/engine/generation/test_pipeline_{sd3_5,wan_2_1,cosmos}.py``,
``tests/models/test_diffusion_policy_module.py``, ``tests/rollouts/test_evaluators.py``)."""

from types import SimpleNamespace

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.models.families.sd3_5.builder import build_sd3_5_runtime_bundle_from_cfg
from visionrl_b200.models.families.sd3_5.executor import SD3_5PipelineExecutor
from visionrl_b200.rollouts.evaluators import SignalRequest
from visionrl_b200.rollouts.evaluators.diffusion import FlowMatchingEvaluator
from visionrl_b200.rollouts.packers.base import RolloutPackContext
from visionrl_b200.rollouts.packers.diffusion import DiffusionRolloutPacker

STEPS = 4


@pytest.fixture(scope="module")
def bundle():
    cfg = load_config("experiment/tiny_dit_grpo", overrides=[f"sampling.num_steps={STEPS}"])
    return build_sd3_5_runtime_bundle_from_cfg(cfg, "cpu", torch.float32), cfg


class _Counting:
    """Counts transformer forwards and prompt encodes of a policy."""

    def __init__(self, policy):
        self.policy, self.forwards, self.encodes = policy, 0, 0
        self._fs, self._enc = policy.forward_step, policy.encode_prompt
        policy.forward_step = self._forward_step
        policy.encode_prompt = self._encode

    def _forward_step(self, *a, **k):
        self.forwards += 1
        return self._fs(*a, **k)

    def _encode(self, *a, **k):
        self.encodes += 1
        return self._enc(*a, **k)

    def restore(self):
        self.policy.forward_step, self.policy.encode_prompt = self._fs, self._enc


def _request(cfg, prompts, n, **extra):
    s = cfg.sampling
    sampling = {"num_steps": STEPS, "guidance_scale": float(s.guidance_scale), "height": int(s.height),
                "width": int(s.width), "max_sequence_length": int(s.max_sequence_length),
                "noise_level": 0.7, "sde_type": "sde", "sample_batch_size": 4, "seed": 11}
    sampling.update(extra)
    return GenerationRequest(request_id="req", family="sd3_5", task="t2i", prompts=prompts,
                             samples_per_prompt=n, sampling=sampling,
                             return_artifacts={"output", "rollout_trajectory_data", "trajectory_latents",
                                               "trajectory_timesteps", "denoising_env"})


def _specs(req):
    return GenerationIdFactory().build_sample_specs(req)


def test_executor_shapes_microbatches_and_encode_counts(bundle):
    b, cfg = bundle
    ex = SD3_5PipelineExecutor(b.policy, sample_batch_size=4)
    counter = _Counting(b.policy)
    try:
        req = _request(cfg, ["a", "b"], 6)                              # 12 samples, batch 4
        out = ex.forward(req, _specs(req))
    finally:
        counter.restore()
    assert out.error is None
    traj = out.rollout_trajectory_data
    assert traj.rollout_log_probs.shape == (12, STEPS)
    assert traj.dit_trajectory.latents.shape[:2] == (12, STEPS)
    assert traj.dit_trajectory.timesteps.shape == (12, STEPS)
    assert out.metrics.micro_batches == 4                               # per prompt: 4 + 2
    assert counter.forwards == 4 * STEPS and counter.encodes == 2       # one encode per prompt
    assert out.metrics.num_samples == 12 and out.metrics.num_steps == STEPS


def test_seeded_rollouts_are_bitwise_reproducible_and_kl_is_optional(bundle):
    b, cfg = bundle
    ex = SD3_5PipelineExecutor(b.policy, sample_batch_size=4)
    req = _request(cfg, ["a", "b"], 4)
    one, two = ex.forward(req, _specs(req)), ex.forward(req, _specs(req))
    la, lb = (o.rollout_trajectory_data.dit_trajectory.latents for o in (one, two))
    assert torch.equal(la, lb)
    assert torch.equal(one.rollout_trajectory_data.rollout_log_probs, two.rollout_trajectory_data.rollout_log_probs)
    other = _request(cfg, ["a", "b"], 4, seed=12)
    assert not torch.equal(la, ex.forward(other, _specs(other)).rollout_trajectory_data.dit_trajectory.latents)
    with_kl = _request(cfg, ["a"], 2, return_kl=True)
    out = ex.forward(with_kl, _specs(with_kl))
    env = out.rollout_trajectory_data.denoising_env.extra
    lp = out.rollout_trajectory_data.rollout_log_probs
    assert torch.equal(env["kl"], lp.abs())
    assert torch.count_nonzero(one.rollout_trajectory_data.denoising_env.extra["kl"]) == 0


def test_same_latent_needs_a_seed(bundle):
    b, cfg = bundle
    ex = SD3_5PipelineExecutor(b.policy, sample_batch_size=4)
    bad = _request(cfg, ["a"], 2, same_latent=True, seed=None)
    with pytest.raises(ValueError, match="same_latent"):
        ex.forward(bad, _specs(bad))
    good = _request(cfg, ["a"], 4, same_latent=True)
    assert ex.forward(good, _specs(good)).error is None


def test_policy_module_registers_only_the_transformer(bundle):
    policy = bundle[0].policy
    assert {n for n, _ in policy.named_children()} == {"transformer"}
    assert all(k.startswith("transformer.") for k in policy.state_dict())
    with pytest.raises(ValueError):
        policy.load_trainable_state({"vae.weight": torch.zeros(1)})
    with pytest.raises(ValueError):
        policy.load_trainable_state({})
    assert set(policy.trainable_modules) == {"transformer"}


def test_evaluator_replays_through_the_policy_and_uses_adapter_off_reference(bundle):
    b, cfg = bundle
    policy = b.policy
    ex = SD3_5PipelineExecutor(policy, sample_batch_size=4)
    req = _request(cfg, ["a"], 4)
    out = ex.forward(req, _specs(req))
    packer = DiffusionRolloutPacker(error_prefix="SD3.5")
    ctx = RolloutPackContext(metadata={}, device=torch.device("cpu"), kl_reward=0.0, rescale_to_unit=False)
    import asyncio

    batch = asyncio.new_event_loop().run_until_complete(packer.pack(out, torch.zeros(4), ctx))
    assert batch.observations.shape[:2] == (4, STEPS) and batch.extras["log_probs"].shape == (4, STEPS)
    evaluator = FlowMatchingEvaluator(b.scheduler, noise_level=0.7, sde_type="sde")
    calls, adapter_states = [], []
    replay = policy.replay_forward

    def spy(batch_, idx):
        calls.append(idx)
        layers = [m for m in policy.transformer.modules() if hasattr(m, "adapter_enabled") and m.has_adapter]
        adapter_states.append(all(m.adapter_enabled for m in layers))
        return replay(batch_, idx)

    policy.replay_forward = spy
    try:
        sig = evaluator.evaluate(policy, batch, 1, ref_model=policy,
                                 signal_request=SignalRequest(need_ref=True, need_kl_intermediates=True))
    finally:
        policy.replay_forward = replay
    assert calls == [1, 1] and adapter_states == [True, False]        # second pass with adapters off
    assert torch.allclose(sig.log_prob, batch.extras["log_probs"][:, 1], atol=1e-5)   # rollout == replay
    assert sig.ref_log_prob is not None and sig.prev_sample_mean is not None and sig.std_dev_t is not None
