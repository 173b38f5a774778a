"""Janus-Pro policy, executor and the AR engine pieces on a tiny random-init network (reference
expectations: ``tests/models/test_janus_wrapper.py``, ``test_janus_replay.py``, ``test_ar_cache.py``,
``tests/engine/generation/test_pipeline_janus_pro.py``, ``test_ar_token_scheduler.py``,
``test_ar_chunk_execution.py``)."""

import random
from types import SimpleNamespace

import pytest
import torch

from visionrl_b200.engine.ar import ActiveSequence, ARTokenScheduler
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.microbatching import MicroBatchPlan
from visionrl_b200.models.ar import ar_concat_rows, ar_split_rows
from visionrl_b200.models.families.janus_pro.executor import (JanusProChunkGatherer,
                                                              JanusProPipelineExecutor)
from visionrl_b200.models.families.janus_pro.policy import JanusProConfig, JanusProPolicy

ARCH = {"num_layers": 2, "hidden_size": 64, "num_heads": 2, "ffn_dim": 128, "vocab_size": 128,
        "image_vocab_size": 96, "codebook_dim": 8, "vq_base": 16, "vq_mults": (1, 2), "vq_blocks": 1}


def _policy(use_lora=True):
    cfg = JanusProConfig(model_path="", dtype="float32", use_lora=use_lora, lora_rank=2, lora_alpha=4,
                         image_token_num=9, image_size=32, patch_size=16, random_init=True, arch=ARCH)
    return JanusProPolicy(cfg, device="cpu")


@pytest.fixture(scope="module")
def policy():
    return _policy()


def _request(prompts, n, **sampling):
    base = {"cfg_weight": 3.0, "temperature": 1.0, "image_token_num": 9, "image_size": 32,
            "max_text_length": 12, "seed": 7}
    base.update(sampling)
    return GenerationRequest(request_id="req", family="janus_pro", task="ar_t2i", prompts=prompts,
                             samples_per_prompt=n, sampling=base)


def _specs(request):
    return GenerationIdFactory().build_sample_specs(request)


# ---------------------------------------------------------------------------------- wrapper
def test_image_logits_come_from_gen_head_with_codebook_width(policy):
    hidden = torch.randn(3, 64)
    logits = policy.policy.image_logits(hidden)
    assert logits.shape == (3, 96)                                   # image codebook, not the text vocab
    assert not hasattr(policy.policy, "lm_head")
    assert policy._resolve_vq_latent_channels() == 8


def test_disable_adapter_needs_lora():
    plain = _policy(use_lora=False)
    with pytest.raises(RuntimeError):
        with plain.disable_adapter():
            pass
    with _policy().disable_adapter():
        pass


def test_decode_clamps_to_unit_range(policy):
    tokens = torch.randint(0, 96, (2, 9))
    images = policy.decode_image_tokens(tokens, image_size=32)
    assert images.shape == (2, 3, 32, 32) and images.min() >= -1 and images.max() <= 1
    with pytest.raises(ValueError):
        policy.decode_image_tokens(torch.zeros(1, 8, dtype=torch.long))


def test_only_trunk_adapters_train(policy):
    names = [n for n, p in policy.named_parameters() if p.requires_grad]
    assert names and all("lora_" in n and "language_model" in n for n in names)


# ----------------------------------------------------------------------------------- replay
def test_replay_returns_logprobs_or_logits_with_grad(policy):
    ex = JanusProPipelineExecutor(policy)
    req = _request(["a red cube"], 2)
    out = ex.forward(req, _specs(req))
    batch = SimpleNamespace(observations=out.extra["prompt_input_ids"].unsqueeze(1),
                            actions=out.extra["token_ids"],
                            extras={"prompt_attention_mask": out.extra["prompt_attention_mask"]},
                            context=out.extra["context"])
    policy.fused_logprob = False
    res = policy.replay_forward(batch)
    assert set(res) == {"logits", "image_token_ids"} and res["logits"].shape == (2, 9, 96)
    assert res["logits"].requires_grad
    lp = torch.log_softmax(res["logits"].float(), -1).gather(-1, out.extra["token_ids"][..., None])[..., 0]
    assert torch.allclose(lp, out.extra["token_log_probs"], atol=1e-4)   # rollout == replay
    policy.fused_logprob = True
    assert not hasattr(ex, "forward_step")


# --------------------------------------------------------------------------------- executor
def test_scheduler_path_equals_black_box_path(policy):
    ex = JanusProPipelineExecutor(policy)
    req = _request(["p0", "p1"], 2)
    a = ex.forward(req, _specs(req))
    sched = _request(["p0", "p1"], 2, use_ar_scheduler=True)
    b = ex.forward(sched, _specs(sched))
    partial = _request(["p0", "p1"], 2, use_ar_scheduler=True, ar_scheduler_batch_size=3)
    c = ex.forward(partial, _specs(partial))
    for other in (b, c):
        assert torch.equal(a.extra["token_ids"], other.extra["token_ids"])
        assert torch.allclose(a.extra["token_log_probs"], other.extra["token_log_probs"], atol=1e-5)
    assert a.output.shape == (4, 3, 32, 32) and torch.all(a.extra["token_mask"] == 1)
    assert a.extra["context"]["cfg_weight"] == 3.0 and a.extra["context"]["temperature"] == 1.0
    again = ex.forward(req, _specs(req))
    assert torch.equal(a.extra["token_ids"], again.extra["token_ids"])     # seed reproducibility


def test_chunks_gathered_out_of_order_are_prompt_major(policy):
    ex = JanusProPipelineExecutor(policy)
    req = _request(["p0", "p1"], 2)
    specs = _specs(req)
    chunks = [ex.forward_chunk(req, MicroBatchPlan(prompt_index=p, prompt=req.prompts[p], sample_start=s,
                                                   sample_count=1)) for p in (0, 1) for s in (0, 1)]
    random.Random(0).shuffle(chunks)
    gatherer = JanusProChunkGatherer()
    assert not hasattr(gatherer, "forward")                         # a pure object, not an executor
    out = gatherer.gather_chunks(req, specs, chunks)
    assert out.extra["token_ids"].shape == (4, 9) and out.metrics.micro_batches == 4
    ordered = sorted(chunks, key=lambda c: (c.prompt_index, c.sample_start))
    assert torch.equal(out.extra["token_ids"], torch.cat([c.token_ids for c in ordered]))
    with pytest.raises(ValueError):
        gatherer.gather_chunks(req, specs, chunks[:3])               # incomplete coverage


# -------------------------------------------------------------------------------- scheduler
def _seq(i, pos=0, max_new=4, family="janus_pro"):
    s = ActiveSequence(request_id="r", sample_id=f"s{i}", family=family, task="ar_t2i",
                       tokenizer_key="janus", dtype="float32", max_new_tokens=max_new)
    for _ in range(pos):
        s.advance()
    return s


def test_token_scheduler_batches_same_key_and_position_only():
    sched = ARTokenScheduler(max_batch_size=2)
    sched.add_many([_seq(0), _seq(1), _seq(2), _seq(3, pos=1), _seq(4, family="nextstep_1")])
    first = sched.pop_batch()
    assert [s.sample_id for s in first.sequences] == ["s0", "s1"]     # capped at max_batch_size
    for s in first.sequences:
        s.advance()
    sched.push_back_unfinished(first)
    keys = set()
    while len(sched):
        batch = sched.pop_batch()
        assert len({(s.family, s.position) for s in batch.sequences}) == 1
        keys.add((batch.sequences[0].family, batch.sequences[0].position))
        for s in batch.sequences:
            for _ in range(s.max_new_tokens - s.position):
                s.advance()
        sched.push_back_unfinished(batch)                            # finished ones are dropped
    assert ("nextstep_1", 0) in keys and ("janus_pro", 1) in keys


# ------------------------------------------------------------------------------- row helpers
def test_kv_row_split_and_concat_preserve_order():
    k, v = torch.arange(12.).view(3, 2, 2), torch.arange(12.).view(3, 2, 2) + 100
    state = {"past_key_values": ((k, v),), "last_hidden": torch.arange(6.).view(3, 2)}
    rows = ar_split_rows(state, 3)
    assert len(rows) == 3 and torch.equal(rows[1]["past_key_values"][0][0], k[1:2])
    merged = ar_concat_rows(rows)
    assert torch.equal(merged["past_key_values"][0][1], v) and torch.equal(merged["last_hidden"],
                                                                          state["last_hidden"])
    with pytest.raises(ValueError):
        ar_split_rows(state, 4)
