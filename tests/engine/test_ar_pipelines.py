"""Executor-level behaviour of the two autoregressive families on tiny random-init networks:
discrete image tokens (Janus-Pro) and continuous tokens with a flow head (NextStep-1).  The
expectations are the ones the reference pins for its executors
(``tests/engine/generation/test_pipeline_janus_pro.py``, ``test_pipeline_nextstep_1.py``): row
counts and order, workload signatures, seeds, the scheduler-driven path, what reaches the model,
metrics, and the reward-image range."""

import pytest
import torch

from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.models.families.janus_pro.executor import JanusProPipelineExecutor
from visionrl_b200.models.families.janus_pro.policy import JanusProConfig, JanusProPolicy
from visionrl_b200.models.families.nextstep_1.executor import NextStep1PipelineExecutor
from visionrl_b200.models.families.nextstep_1.policy import NextStep1Config, NextStep1Policy

JANUS_ARCH = {"num_layers": 2, "hidden_size": 64, "num_heads": 2, "ffn_dim": 128, "vocab_size": 128,
              "image_vocab_size": 96, "codebook_dim": 8, "vq_base": 16, "vq_mults": (1, 2), "vq_blocks": 1}
NEXT_ARCH = {"num_layers": 2, "hidden_size": 64, "num_heads": 2, "ffn_dim": 128, "vocab_size": 128,
             "token_dim": 16, "token_patch": 2, "head_hidden": 32, "head_layers": 2, "vae_base": 8,
             "vae_mults": (1, 2), "vae_blocks": 1}


@pytest.fixture(scope="module")
def janus():
    cfg = JanusProConfig(model_path="", dtype="float32", use_lora=True, lora_rank=2, lora_alpha=4,
                         image_token_num=9, image_size=32, patch_size=16, random_init=True, arch=JANUS_ARCH)
    return JanusProPipelineExecutor(JanusProPolicy(cfg, device="cpu"))


@pytest.fixture(scope="module")
def nextstep():
    cfg = NextStep1Config(model_path="", vae_path="", dtype="float32", use_lora=True, lora_rank=2, lora_alpha=4,
                          image_token_num=4, image_size=16, num_flow_steps=3, random_init=True, arch=NEXT_ARCH)
    return NextStep1PipelineExecutor(NextStep1Policy(cfg, device="cpu"))


def _janus_request(prompts=("a cat", "a dog"), n=4, **sampling):
    base = {"cfg_weight": 3.0, "temperature": 1.0, "image_token_num": 9, "image_size": 32,
            "max_text_length": 12, "seed": 11}
    base.update(sampling)
    return GenerationRequest(request_id="jr", family="janus_pro", task="ar_t2i", prompts=list(prompts),
                             samples_per_prompt=n, sampling=base)


def _next_request(prompts=("a cat", "a dog"), n=4, **sampling):
    base = {"cfg_scale": 2.0, "num_flow_steps": 3, "noise_level": 0.8, "image_token_num": 4, "image_size": 16,
            "max_text_length": 12, "seed": 5}
    base.update(sampling)
    return GenerationRequest(request_id="nr", family="nextstep_1", task="ar_t2i", prompts=list(prompts),
                             samples_per_prompt=n, sampling=base)


def _run(executor, request):
    return executor.forward(request, GenerationIdFactory().build_sample_specs(request))


# ------------------------------------------------------------------------------- discrete tokens
def test_janus_two_prompts_four_samples_give_eight_prompt_major_rows(janus):
    out = _run(janus, _janus_request())
    assert out.output.shape == (8, 3, 32, 32)
    assert out.extra["token_ids"].shape == (8, 9) and out.extra["token_ids"].dtype == torch.long
    assert out.extra["token_log_probs"].shape == (8, 9)
    assert [s.prompt_index for s in out.sample_specs] == [0] * 4 + [1] * 4
    assert [s.sample_index for s in out.sample_specs] == list(range(4)) * 2
    assert int(out.extra["token_ids"].min()) >= 0 and int(out.extra["token_ids"].max()) < 96
    assert bool((out.extra["token_log_probs"] <= 0).all())
    assert torch.all(out.extra["token_mask"] == 1) and out.extra["token_mask"].shape == (8, 9)
    assert float(out.output.min()) >= -1.0 and float(out.output.max()) <= 1.0


def test_janus_workload_signature_follows_the_request(janus):
    sig = janus.workload_signature(_janus_request(n=4, max_new_tokens=9))
    other = janus.workload_signature(_janus_request(n=4, max_new_tokens=16))
    assert (sig.family, sig.task, sig.max_new_tokens) == ("janus_pro", "ar_t2i", 9)
    assert sig == janus.workload_signature(_janus_request(n=2, max_new_tokens=9)) and sig != other


def test_janus_seed_decides_the_tokens(janus):
    a, b = _run(janus, _janus_request()), _run(janus, _janus_request())
    c = _run(janus, _janus_request(seed=12))
    assert torch.equal(a.extra["token_ids"], b.extra["token_ids"])
    assert torch.equal(a.extra["token_log_probs"], b.extra["token_log_probs"])
    assert not torch.equal(a.extra["token_ids"], c.extra["token_ids"])


def test_janus_partial_scheduler_batches_are_complete_and_deterministic(janus):
    whole = _run(janus, _janus_request(n=3))
    parts = _run(janus, _janus_request(n=3, use_ar_scheduler=True, ar_scheduler_batch_size=4))
    again = _run(janus, _janus_request(n=3, use_ar_scheduler=True, ar_scheduler_batch_size=4))
    assert parts.extra["token_ids"].shape == (6, 9)
    assert torch.equal(parts.extra["token_ids"], again.extra["token_ids"])
    assert torch.equal(parts.extra["token_ids"], whole.extra["token_ids"])
    assert torch.allclose(parts.extra["token_log_probs"], whole.extra["token_log_probs"], atol=1e-5)


def test_janus_guidance_and_temperature_reach_the_sampler(janus):
    base = _run(janus, _janus_request())
    hot = _run(janus, _janus_request(temperature=2.5))
    unguided = _run(janus, _janus_request(cfg_weight=1.0))
    assert base.extra["context"]["cfg_weight"] == 3.0 and hot.extra["context"]["temperature"] == 2.5
    assert not torch.allclose(base.extra["token_log_probs"], hot.extra["token_log_probs"])
    assert not torch.allclose(base.extra["token_log_probs"], unguided.extra["token_log_probs"])
    # a hotter distribution is flatter: the chosen tokens are, on average, less likely
    assert float(hot.extra["token_log_probs"].mean()) < float(base.extra["token_log_probs"].mean())


def test_janus_metrics_describe_the_request(janus):
    m = _run(janus, _janus_request(n=2)).metrics
    assert (m.num_prompts, m.num_samples, m.num_steps, m.micro_batches) == (2, 4, 9, 1)


# ----------------------------------------------------------------------------- continuous tokens
def test_nextstep_rows_tokens_noise_and_replay_context(nextstep):
    out = _run(nextstep, _next_request())
    assert out.output.shape == (8, 3, 16, 16)
    assert out.extra["tokens"].shape == (8, 4, 16) and out.extra["saved_noise"].shape == (8, 4, 16)
    assert out.extra["log_probs"].shape == (8, 4) and torch.isfinite(out.extra["log_probs"]).all()
    for key in ("prompt_input_ids", "prompt_attention_mask", "uncond_input_ids", "uncond_attention_mask"):
        assert out.extra[key].shape[0] == 8
    # no DiT trajectory for a continuous-token rollout; the record carries the log-probabilities only
    traj = out.rollout_trajectory_data
    assert traj.dit_trajectory is None and traj.denoising_env is None
    assert torch.equal(traj.rollout_log_probs, out.extra["log_probs"])
    ctx = out.extra["context"]
    assert (ctx["cfg_scale"], ctx["num_flow_steps"], ctx["noise_level"]) == (2.0, 3, 0.8)
    assert (out.metrics.num_prompts, out.metrics.num_samples, out.metrics.num_steps) == (2, 8, 4)


def test_nextstep_seeds_and_scheduler_paths(nextstep):
    a, b = _run(nextstep, _next_request(n=2)), _run(nextstep, _next_request(n=2))
    c = _run(nextstep, _next_request(n=2, seed=6))
    assert torch.equal(a.extra["tokens"], b.extra["tokens"])
    assert not torch.equal(a.extra["tokens"], c.extra["tokens"])
    sched = _run(nextstep, _next_request(n=2, use_ar_scheduler=True))
    assert torch.equal(a.extra["tokens"], sched.extra["tokens"])      # the scheduled path is the same computation
    assert torch.equal(a.extra["log_probs"], sched.extra["log_probs"])
    partial = _run(nextstep, _next_request(n=2, use_ar_scheduler=True, ar_scheduler_batch_size=3))
    twice = _run(nextstep, _next_request(n=2, use_ar_scheduler=True, ar_scheduler_batch_size=3))
    assert partial.extra["tokens"].shape == (4, 4, 16)
    assert torch.equal(partial.extra["tokens"], twice.extra["tokens"])


def test_nextstep_reward_images_are_unit_range_only_when_asked(nextstep):
    unit = _run(nextstep, _next_request(n=1, rescale_to_unit=True))
    imgs = unit.extra["images_for_reward"]
    assert float(imgs.min()) >= 0.0 and float(imgs.max()) <= 1.0
    assert torch.allclose(imgs, ((unit.output + 1.0) * 0.5).clamp(0.0, 1.0))
    native = _run(nextstep, _next_request(n=1, rescale_to_unit=False))
    assert torch.equal(native.extra["images_for_reward"], native.output)


def test_nextstep_one_sampling_call_and_one_decode_per_request(nextstep, monkeypatch):
    calls = {"sample": 0, "decode": 0}
    model = nextstep.model
    sample, decode = model.sample_image_tokens, model.decode_image_tokens

    def counted_sample(*a, **k):
        calls["sample"] += 1
        return sample(*a, **k)

    def counted_decode(*a, **k):
        calls["decode"] += 1
        return decode(*a, **k)

    monkeypatch.setattr(model, "sample_image_tokens", counted_sample, raising=False)
    monkeypatch.setattr(model, "decode_image_tokens", counted_decode, raising=False)
    _run(nextstep, _next_request(n=4))
    assert calls == {"sample": 1, "decode": 1}
