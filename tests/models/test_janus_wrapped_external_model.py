"""The Janus policy around an externally loaded model: a small ``transformers`` LLaMA as the
trunk, so that the cache handling meets a real cache object (reference contract:
``vrl/models/families/janus_pro/policy.py:177-224``)."""

from types import SimpleNamespace

import pytest
import torch
from torch import nn

transformers = pytest.importorskip("transformers")

from visionrl_b200.models.families.janus_pro.policy import JanusProConfig, JanusProPolicy
from visionrl_b200.models.families.janus_pro.wrapped import WrappedJanusProPolicy, host_linear_layers
from visionrl_b200.models.nn.layers import LoRALinear

HIDDEN, VOCAB, IMG_VOCAB, CODE = 32, 50, 40, 6


class _VQ(nn.Module):
    def __init__(self):
        super().__init__()
        self.quantize = nn.Module()
        self.quantize.embedding = nn.Embedding(IMG_VOCAB, CODE)
        self.seen = None

    def decode_code(self, ids, shape):
        self.seen = list(shape)
        b, _, h, w = shape
        return torch.full((b, 3, h * 16, w * 16), 3.0)


class _External(nn.Module):
    def __init__(self):
        super().__init__()
        cfg = transformers.LlamaConfig(hidden_size=HIDDEN, intermediate_size=64, num_hidden_layers=2,
                                       num_attention_heads=4, num_key_value_heads=2, vocab_size=VOCAB,
                                       max_position_embeddings=64)
        self.language_model = transformers.LlamaForCausalLM(cfg)
        self.gen_vision_model = _VQ()
        self.gen_head = nn.Linear(HIDDEN, IMG_VOCAB)
        self.gen_embed = nn.Embedding(IMG_VOCAB, HIDDEN)

    def prepare_gen_img_embeds(self, ids):
        return self.gen_embed(ids)


def _policy(use_lora=False, **cfg):
    torch.manual_seed(0)
    config = JanusProConfig(use_lora=use_lora, lora_rank=4, lora_alpha=8, cfg_weight=3.0,
                            image_token_num=6, **cfg)
    return JanusProPolicy(config, mmgpt=_External().eval(), processor=object())


def _prompts(policy, b=3, l_text=5, seed=1):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, VOCAB, (b, l_text), generator=g)
    unc = torch.randint(0, VOCAB, (b, l_text), generator=g)
    mask = torch.ones(b, l_text, dtype=torch.long)
    return ids, policy.embed_text(ids), policy.embed_text(unc), mask


def test_constructor_dispatches_on_mmgpt():
    policy = _policy()
    assert isinstance(policy, WrappedJanusProPolicy) and isinstance(policy, JanusProPolicy)
    assert policy.trainable_param_count() == 0 and policy.has_lora_adapter is False
    with pytest.raises(ValueError, match="processor"):
        JanusProPolicy(JanusProConfig(use_lora=False), mmgpt=_External())
    with pytest.raises(RuntimeError, match="Janus"):
        JanusProPolicy(JanusProConfig(use_lora=False), mmgpt=nn.Linear(2, 2), processor=object())
    with pytest.raises(RuntimeError, match="no PEFT adapter"):
        policy.disable_adapter()


def test_sampled_log_probs_equal_the_teacher_forced_replay():
    policy = _policy()
    ids, cond, uncond, mask = _prompts(policy)
    tokens, log_probs = policy.sample_image_tokens(cond, uncond, mask, mask,
                                                   generator=torch.Generator().manual_seed(7))
    assert tokens.shape == (3, 6) and tokens.dtype == torch.long and log_probs.dtype == torch.float32
    batch = SimpleNamespace(observations=ids.unsqueeze(1), actions=tokens,
                            extras={"prompt_attention_mask": mask})
    out = policy.replay_forward(batch)
    assert set(out) == {"logits", "image_token_ids"}
    replayed = torch.log_softmax(out["logits"].float(), dim=-1).gather(-1, tokens[..., None])[..., 0]
    torch.testing.assert_close(replayed, log_probs, atol=2e-5, rtol=1e-5)


def test_token_scheduled_sampling_of_row_subsets_matches_black_box_sampling():
    policy = _policy()
    _, cond, uncond, mask = _prompts(policy)
    whole = policy.sample_image_tokens(cond, uncond, mask, mask, generator=torch.Generator().manual_seed(3))
    state = policy.init_ar_state(cond, uncond, mask, mask, generator=torch.Generator().manual_seed(3))

    def seqs(rows, position):
        return [SimpleNamespace(metadata={"row_index": r}, position=position, sample_id=f"s{r}") for r in rows]

    # all rows take the first step together (one batched cache), then the groups drift apart
    policy.step_ar(state, seqs([0, 1, 2], 0))
    for position in range(1, 6):
        policy.step_ar(state, seqs([1], position))
    for position in range(1, 6):
        result = policy.step_ar(state, seqs([2, 0], position))
        assert result.sequence_ids == ["s2", "s0"] and result.positions == [position, position]
    tokens, log_probs = policy.finalize_ar_state(state)
    assert torch.equal(tokens, whole[0])
    torch.testing.assert_close(log_probs, whole[1], atol=2e-5, rtol=1e-5)
    with pytest.raises(ValueError, match="already produced"):
        policy.step_ar(state, seqs([0], 6))


def test_lora_is_hosted_on_the_external_linear_layers():
    policy = _policy(use_lora=True)
    hosted = [m for m in policy.language_model.modules() if isinstance(m, LoRALinear)]
    assert len(hosted) == 2 * 4 and all(m.has_adapter for m in hosted)
    trainable = [n for n, p in policy.named_parameters() if p.requires_grad]
    assert trainable and all(n.endswith(("lora_A", "lora_B")) for n in trainable)
    assert policy.has_lora_adapter is True
    ids, cond, _, mask = _prompts(policy)
    tokens = torch.randint(0, IMG_VOCAB, (3, 6))
    base = policy.forward_image_logits(cond, mask, tokens)
    with torch.no_grad():
        for m in hosted:
            m.lora_B.normal_(std=0.05)
    tuned = policy.forward_image_logits(cond, mask, tokens)
    assert not torch.allclose(tuned, base, atol=1e-4)
    with policy.disable_adapter():
        off = policy.forward_image_logits(cond, mask, tokens)
    torch.testing.assert_close(off, base, atol=1e-5, rtol=1e-5)
    tuned.float().logsumexp(-1).sum().backward()
    assert all(m.lora_A.grad is not None and m.lora_B.grad is not None for m in hosted)


def test_hosting_shares_the_parameters():
    block = nn.Sequential()
    block.q_proj = nn.Linear(4, 4)
    block.other = nn.Linear(4, 4)
    weight = block.q_proj.weight
    assert host_linear_layers(block, ("q_proj",)) == ["q_proj"]
    assert isinstance(block.q_proj, LoRALinear) and block.q_proj.weight is weight
    assert type(block.other) is nn.Linear


def test_codebook_width_comes_from_the_override_or_the_live_table():
    policy = _policy()
    images = policy.decode_image_tokens(torch.zeros(2, 4, dtype=torch.long))
    assert policy.vq_model.seen == [2, CODE, 2, 2]
    assert images.shape == (2, 3, 32, 32) and float(images.max()) == 1.0
    policy.config.vq_latent_channels = 9
    policy.decode_image_tokens(torch.zeros(1, 4, dtype=torch.long))
    assert policy.vq_model.seen[1] == 9
    policy.config.vq_latent_channels = -2
    with pytest.raises(RuntimeError, match="positive int"):
        policy.decode_image_tokens(torch.zeros(1, 4, dtype=torch.long))
    policy.config.vq_latent_channels = None
    del policy.vq_model.quantize
    with pytest.raises(RuntimeError, match="vq_latent_channels"):
        policy.decode_image_tokens(torch.zeros(1, 4, dtype=torch.long))


# ------------------------------------------------------------------ through the pipeline executor
class _Tokenizer:
    """Callable with the Hugging Face tokenizer interface the executor uses: fixed-length ids from
    character codes, left as zeros (the pad id) beyond the text."""

    pad_token_id = 0

    def __call__(self, texts, return_tensors="pt", padding="max_length", truncation=True, max_length=8):
        ids = torch.zeros(len(texts), max_length, dtype=torch.long)
        mask = torch.zeros(len(texts), max_length, dtype=torch.long)
        for row, text in enumerate(texts):
            codes = [1 + (ord(ch) % (VOCAB - 1)) for ch in text][-max_length:]
            ids[row, : len(codes)] = torch.tensor(codes)
            mask[row, : len(codes)] = 1
        return {"input_ids": ids, "attention_mask": mask}


def _executor():
    from visionrl_b200.models.families.janus_pro.executor import JanusProPipelineExecutor

    torch.manual_seed(0)
    config = JanusProConfig(use_lora=True, lora_rank=4, lora_alpha=8, image_token_num=4)
    policy = JanusProPolicy(config, mmgpt=_External().eval(), processor=SimpleNamespace(tokenizer=_Tokenizer()))
    return JanusProPipelineExecutor(policy)


def _request(**sampling):
    from visionrl_b200.engine.core.types import GenerationRequest

    base = {"cfg_weight": 2.0, "temperature": 1.0, "image_token_num": 4, "image_size": 32,
            "max_text_length": 24, "seed": 5}
    base.update(sampling)
    return GenerationRequest(request_id="w", family="janus_pro", task="ar_t2i", prompts=["a cat", "two dogs"],
                             samples_per_prompt=2, sampling=base)


def test_executor_serves_the_wrapped_policy_on_both_sampling_paths():
    from visionrl_b200.engine.core.worker import GenerationIdFactory

    executor = _executor()

    def run(request):
        return executor.forward(request, GenerationIdFactory().build_sample_specs(request))

    whole = run(_request())
    assert whole.output.shape == (4, 3, 32, 32)
    assert whole.extra["token_ids"].shape == (4, 4) and bool((whole.extra["token_log_probs"] <= 0).all())
    assert torch.equal(run(_request()).extra["token_ids"], whole.extra["token_ids"])
    parts = run(_request(use_ar_scheduler=True, ar_scheduler_batch_size=3))
    assert torch.equal(parts.extra["token_ids"], whole.extra["token_ids"])
    torch.testing.assert_close(parts.extra["token_log_probs"], whole.extra["token_log_probs"],
                               atol=2e-5, rtol=1e-5)
    # the rollout's log-probabilities are what the training-time replay recomputes
    batch = SimpleNamespace(observations=whole.extra["prompt_input_ids"].unsqueeze(1),
                            actions=whole.extra["token_ids"],
                            extras={"prompt_attention_mask": whole.extra["prompt_attention_mask"]})
    out = executor.model.replay_forward(batch)
    replayed = torch.log_softmax(out["logits"].float(), -1).gather(-1, whole.extra["token_ids"][..., None])[..., 0]
    torch.testing.assert_close(replayed, whole.extra["token_log_probs"], atol=2e-5, rtol=1e-5)
