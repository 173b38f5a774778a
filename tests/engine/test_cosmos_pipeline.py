"""The Cosmos Predict2 Video2World executor over a tiny random-init network on CPU: the first
latent frame is the conditioning frame and never moves, the reference image comes from the
constructor unless the request carries one, chunks gather to what one forward gives, and the
replay through the evaluator reproduces the rollout's log-probabilities (reference expectations:
``tests/engine/generation/test_pipeline_cosmos.py``)."""

import asyncio

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.engine.core.types import GenerationRequest, WorkloadSignature
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.gather import DiffusionChunkGatherer
from visionrl_b200.engine.microbatching import MicroBatchPlan

STEPS = 3
TINY = ["model.random_init=true", "model.use_lora=false", "+model.dtype=float32",
        "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
        "model.arch.ffn_dim=128", "model.arch.text_dim=32", "model.arch.freq_dim=32",
        f"sampling.num_steps={STEPS}", "sampling.width=32", "sampling.height=32", "sampling.num_frames=5",
        "sampling.max_sequence_length=8", "distributed.rollout.gpus_per_worker=0"]


def _request(prompts, n, metadata=None, **extra):
    sampling = {"num_steps": STEPS, "guidance_scale": 3.0, "height": 32, "width": 32, "num_frames": 5,
                "max_sequence_length": 8, "noise_level": 0.7, "sde_type": "sde", "sample_batch_size": 2,
                "seed": 5}
    sampling.update(extra)
    return GenerationRequest(request_id="req", family="cosmos", task="v2w", prompts=prompts,
                             samples_per_prompt=n, sampling=sampling, metadata=metadata or {})


@pytest.fixture(scope="module")
def cosmos():
    from visionrl_b200.models.families.cosmos.builder import build_cosmos_predict2_runtime_bundle_from_cfg
    from visionrl_b200.models.families.cosmos.executor import CosmosPipelineExecutor

    cfg = load_config("experiment/cosmos_predict2_2b_grpo", overrides=TINY)
    bundle = build_cosmos_predict2_runtime_bundle_from_cfg(cfg, "cpu", torch.float32)
    return bundle, CosmosPipelineExecutor(bundle.policy, sample_batch_size=2, reference_image="ctor.png")


def _run(ex, req):
    return ex.forward(req, GenerationIdFactory().build_sample_specs(req))


def test_two_prompts_four_samples_give_eight_video_rows_and_the_conditioning_frame_stays(cosmos):
    _, ex = cosmos
    out = _run(ex, _request(["a", "b"], 4))
    traj = out.rollout_trajectory_data
    lat = traj.dit_trajectory.latents
    assert lat.ndim == 6 and lat.shape[:2] == (8, STEPS)                    # [B, T, C, F, h, w]
    assert traj.rollout_log_probs.shape == (8, STEPS) and bool(torch.isfinite(traj.rollout_log_probs).all())
    assert out.output.ndim == 5 and out.output.shape[0] == 8
    assert out.metrics.micro_batches == 4 and out.metrics.num_samples == 8 and out.metrics.num_prompts == 2
    assert [s.prompt_index for s in out.sample_specs] == [0, 0, 0, 0, 1, 1, 1, 1]
    init = traj.denoising_env.extra["training_extras"]["init_latents"]
    assert init.shape[0] == 8 and bool((init[:, :, 1:] == 0).all())       # only the first latent frame conditions
    assert bool((init[:, :, 0].abs().sum((1, 2, 3)) > 0).all())
    assert traj.denoising_env.extra["videos"].shape[0] == 8


def test_workload_signature_follows_the_request(cosmos):
    _, ex = cosmos
    a = ex.workload_signature(_request(["a"], 2))
    assert isinstance(a, WorkloadSignature) and a == ex.workload_signature(_request(["other"], 2))
    assert a != ex.workload_signature(_request(["a"], 2, num_frames=9))
    assert a != ex.workload_signature(_request(["a"], 2, height=64))


def test_seed_decides_the_rollout_and_kl_is_optional(cosmos):
    _, ex = cosmos
    one, two = _run(ex, _request(["a"], 2)), _run(ex, _request(["a"], 2))
    lat = lambda o: o.rollout_trajectory_data.dit_trajectory.latents          # noqa: E731
    assert torch.equal(lat(one), lat(two))
    assert not torch.equal(lat(one), lat(_run(ex, _request(["a"], 2, seed=6))))
    kl_off = _run(ex, _request(["a"], 2, return_kl=False)).rollout_trajectory_data
    kl_on = _run(ex, _request(["a"], 2, return_kl=True)).rollout_trajectory_data
    assert torch.allclose(kl_on.denoising_env.extra["kl"], kl_on.rollout_log_probs.abs())
    assert float(kl_off.denoising_env.extra["kl"].abs().sum()) == 0.0


def test_reference_image_changes_the_rollout_and_the_request_wins_over_the_constructor(cosmos):
    bundle, ex = cosmos
    from visionrl_b200.models.families.cosmos.executor import CosmosPipelineExecutor

    lat = lambda o: o.rollout_trajectory_data.dit_trajectory.latents          # noqa: E731
    ctor = _run(ex, _request(["a"], 2))
    other = CosmosPipelineExecutor(bundle.policy, sample_batch_size=2, reference_image="other.png")
    assert not torch.equal(lat(ctor), lat(_run(other, _request(["a"], 2))))
    # the request's image overrides whatever the executor was built with
    same = _run(other, _request(["a"], 2, metadata={"reference_image": "ctor.png"}))
    assert torch.equal(lat(ctor), lat(same))


def test_chunks_gather_to_the_same_batch_as_one_forward(cosmos):
    _, ex = cosmos
    req = _request(["a"], 3)
    specs = GenerationIdFactory().build_sample_specs(req)
    whole = ex.forward(req, specs)
    chunks = [ex.forward_chunk(req, MicroBatchPlan(prompt_index=0, prompt="a", sample_start=s, sample_count=c))
              for s, c in ((0, 2), (2, 1))]
    gathered = DiffusionChunkGatherer(model_family="cosmos", respect_cfg_flag=False).gather_chunks(req, specs, chunks)
    assert torch.equal(gathered.rollout_trajectory_data.rollout_log_probs,
                       whole.rollout_trajectory_data.rollout_log_probs)
    assert torch.equal(gathered.output, whole.output)


def test_replay_reproduces_the_rollout_log_probs_and_carries_the_conditioning(cosmos):
    from visionrl_b200.rollouts.evaluators.diffusion import FlowMatchingEvaluator
    from visionrl_b200.rollouts.packers.base import RolloutPackContext
    from visionrl_b200.rollouts.packers.diffusion import DiffusionRolloutPacker

    bundle, ex = cosmos
    out = _run(ex, _request(["a"], 2))
    ctx = RolloutPackContext(metadata={}, device=torch.device("cpu"), kl_reward=0.0, rescale_to_unit=False)
    batch = asyncio.new_event_loop().run_until_complete(
        DiffusionRolloutPacker(error_prefix="Cosmos").pack(out, torch.zeros(2), ctx))
    assert batch.extras["init_latents"].shape[0] == 2
    for key in ("cond_indicator", "uncond_indicator", "cond_mask", "padding_mask", "fps"):
        assert key in batch.context
    ind = batch.context["cond_indicator"]
    assert float(ind[0, 0, 0]) == 1.0 and float(ind[0, 0, 1:].sum()) == 0.0
    # the denoised prediction of the conditioning frame is the reference latent itself, with and
    # without the prompt (the frame is re-applied after the network)
    state = bundle.policy.restore_eval_state(batch.extras, batch.context, batch.observations[:, 0], 0)
    with torch.no_grad():
        pred = bundle.policy.forward_step(state, 0)
    init = batch.extras["init_latents"]
    assert torch.allclose(pred["noise_pred_cond"][:, :, 0], init[:, :, 0], atol=1e-6)
    assert torch.allclose(pred["noise_pred_uncond"][:, :, 0], init[:, :, 0], atol=1e-6)
    assert not torch.allclose(pred["noise_pred_cond"][:, :, 1:], init[:, :, 1:], atol=1e-3)
    ev = FlowMatchingEvaluator(bundle.scheduler, noise_level=0.7, sde_type="sde")
    for j in range(STEPS):
        sig = ev.evaluate(bundle.policy, batch, j)
        assert torch.allclose(sig.log_prob, batch.extras["log_probs"][:, j], atol=1e-4)
