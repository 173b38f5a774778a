"""Prompt conditioning from local pipeline directories: tiny random ``transformers`` text
encoders are saved in the pipeline layout, the native prompt encoders load them as they are, and
their output must equal the conditioning computed with the ``transformers`` modules the way the
public pipelines do it (Wan: masked UMT5 with zeros after the prompt; SD3: two CLIP towers'
second-to-last states + projected pooled states, then T5)."""

import json
import os

import pytest
import torch
import torch.nn.functional as F

from visionrl_b200.config.loader import load_config
from visionrl_b200.models.nn.prompt_encoders import CLIP_TOKENS, SD3PromptEncoder, UMT5PromptEncoder

transformers = pytest.importorskip("transformers")
tokenizers = pytest.importorskip("tokenizers")


def _bytes_to_unicode():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs, extra = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + extra)
            extra += 1
    return [chr(c) for c in cs]


def _save_clip(root, name, tok_name, hidden, proj, seed):
    from safetensors.torch import save_file

    chars = _bytes_to_unicode()
    vocab = {t: i for i, t in enumerate(chars + [c + "</w>" for c in chars] + ["<|startoftext|>", "<|endoftext|>"])}
    os.makedirs(root / tok_name)
    (root / tok_name / "vocab.json").write_text(json.dumps(vocab))
    (root / tok_name / "merges.txt").write_text("#version: 0.2\n")
    torch.manual_seed(seed)
    eos = vocab["<|endoftext|>"]
    cfg = transformers.CLIPTextConfig(vocab_size=len(vocab), hidden_size=hidden, intermediate_size=2 * hidden,
                                      num_hidden_layers=3, num_attention_heads=2, max_position_embeddings=CLIP_TOKENS,
                                      hidden_act="quick_gelu" if seed % 2 else "gelu", projection_dim=proj,
                                      bos_token_id=vocab["<|startoftext|>"], eos_token_id=eos, pad_token_id=eos)
    model = transformers.CLIPTextModelWithProjection(cfg).eval()
    os.makedirs(root / name)
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, str(root / name / "model.safetensors"))
    (root / name / "config.json").write_text(json.dumps(cfg.to_dict()))
    return model, transformers.CLIPTokenizer.from_pretrained(str(root / tok_name))


def _save_t5(root, name, tok_name, width, kind, seed):
    from safetensors.torch import save_file
    from tokenizers import Tokenizer, models, pre_tokenizers, processors

    words = ["<pad>", "</s>", "<unk>"] + [chr(c) for c in range(97, 123)] + [" ", ","]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    tok.post_processor = processors.TemplateProcessing(single="$A </s>", special_tokens=[("</s>", 1)])
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", eos_token="</s>",
                                                unk_token="<unk>")
    fast.save_pretrained(str(root / tok_name))
    torch.manual_seed(seed)
    common = dict(vocab_size=len(words), d_model=width, d_kv=8, d_ff=2 * width, num_layers=2, num_heads=4,
                  relative_attention_num_buckets=8, relative_attention_max_distance=16, dropout_rate=0.0,
                  feed_forward_proj="gated-gelu")
    if kind == "umt5":
        cfg = transformers.UMT5Config(**common)
        model = transformers.UMT5EncoderModel(cfg).eval()
    else:
        cfg = transformers.T5Config(**common)
        model = transformers.T5EncoderModel(cfg).eval()
    os.makedirs(root / name)
    save_file({k: v.contiguous() for k, v in model.state_dict().items() if k != "encoder.embed_tokens.weight"},
              str(root / name / "model.safetensors"))
    (root / name / "config.json").write_text(json.dumps(cfg.to_dict()))
    return model, transformers.AutoTokenizer.from_pretrained(str(root / tok_name))


PROMPT = "a red fox, at dusk"


def test_wan_style_conditioning_is_masked_umt5_with_zeros_after_the_prompt(tmp_path):
    model, tok = _save_t5(tmp_path, "text_encoder", "tokenizer", 32, "umt5", 0)
    encoder = UMT5PromptEncoder.from_directory(str(tmp_path))
    context, pooled = encoder([PROMPT, "boats"], 24, "cpu", torch.float32)
    assert context.shape == (2, 24, 32) and pooled is None
    batch = tok([PROMPT], padding="max_length", max_length=24, truncation=True, return_tensors="pt")
    with torch.no_grad():
        want = model(input_ids=batch["input_ids"], attention_mask=batch["attention_mask"]).last_hidden_state[0]
    n = int(batch["attention_mask"].sum())
    assert n == len(PROMPT) + 1
    assert torch.allclose(context[0, :n], want[:n], atol=3e-5)
    assert float(context[0, n:].abs().max()) == 0.0
    # the second call is served from the cache: same tensors, nothing re-encoded
    again, _ = encoder([PROMPT], 24, "cpu", torch.float32)
    assert torch.equal(again[0], context[0]) and len(encoder._host) == 2


def test_sd3_style_conditioning_follows_the_public_recipe(tmp_path):
    clip_l, tok_l = _save_clip(tmp_path, "text_encoder", "tokenizer", 64, 24, 1)
    clip_g, tok_g = _save_clip(tmp_path, "text_encoder_2", "tokenizer_2", 128, 40, 2)
    t5, tok_t5 = _save_t5(tmp_path, "text_encoder_3", "tokenizer_3", 256, "t5", 3)
    encoder = SD3PromptEncoder.from_directory(str(tmp_path), joint_dim=256)
    t5_tokens = 20
    context, pooled = encoder([PROMPT], CLIP_TOKENS + t5_tokens, "cpu", torch.float32)
    assert context.shape == (1, CLIP_TOKENS + t5_tokens, 256) and pooled.shape == (1, 64)

    def clip_part(model, tok):
        ids = tok([PROMPT], padding="max_length", max_length=CLIP_TOKENS, truncation=True, return_tensors="pt")["input_ids"]
        with torch.no_grad():
            out = model(input_ids=ids, output_hidden_states=True)
        return out.hidden_states[-2][0], out.text_embeds[0]

    (h_l, p_l), (h_g, p_g) = clip_part(clip_l, tok_l), clip_part(clip_g, tok_g)
    clip = F.pad(torch.cat([h_l, h_g], dim=-1), (0, 256 - 192))
    ids = tok_t5([PROMPT], padding="max_length", max_length=t5_tokens, truncation=True, return_tensors="pt")["input_ids"]
    with torch.no_grad():
        tail = t5(input_ids=ids).last_hidden_state[0]
    assert torch.allclose(context[0, :CLIP_TOKENS], clip, atol=3e-5)
    assert torch.allclose(context[0, CLIP_TOKENS:], tail, atol=3e-5)
    assert torch.allclose(pooled[0], torch.cat([p_l, p_g]), atol=3e-5)

    # without the third encoder that part of the context is zeros
    import shutil

    shutil.rmtree(tmp_path / "text_encoder_3")
    two = SD3PromptEncoder.from_directory(str(tmp_path), joint_dim=256)
    context2, _ = two([PROMPT], CLIP_TOKENS + 5, "cpu", torch.float32)
    assert torch.allclose(context2[0, :CLIP_TOKENS], clip, atol=3e-5) and float(context2[0, CLIP_TOKENS:].abs().max()) == 0.0
    with pytest.raises(ValueError, match="cannot hold"):
        two.encode(PROMPT, CLIP_TOKENS - 1)


def test_policies_take_the_real_encoders_from_the_config(tmp_path):
    from visionrl_b200.models.families.sd3_5.builder import build_sd3_5_runtime_bundle_from_cfg
    from visionrl_b200.models.families.wan_2_1.builder import build_wan_2_1_runtime_bundle_from_cfg

    sd3_dir, wan_dir = tmp_path / "sd3", tmp_path / "wan"
    sd3_dir.mkdir()
    wan_dir.mkdir()
    _save_clip(sd3_dir, "text_encoder", "tokenizer", 64, 24, 1)
    _save_clip(sd3_dir, "text_encoder_2", "tokenizer_2", 128, 40, 2)
    _save_t5(sd3_dir, "text_encoder_3", "tokenizer_3", 256, "t5", 3)
    _save_t5(wan_dir, "text_encoder", "tokenizer", 32, "umt5", 0)

    cfg = load_config("experiment/sd3_5_ocr_grpo", overrides=[
        "model.random_init=true", "model.use_lora=false", "model.arch.num_layers=2", "model.arch.hidden_size=64",
        "model.arch.num_heads=2", "model.arch.context_dim=256", "model.arch.pooled_dim=64", "model.arch.in_channels=4",
        "sampling.height=32", "sampling.width=32", f"+model.text_encoder.path={sd3_dir}"])
    policy = build_sd3_5_runtime_bundle_from_cfg(cfg, "cpu", torch.float32).policy
    assert isinstance(policy.backend_handle.text, SD3PromptEncoder)
    enc = policy.encode_prompt([PROMPT], max_sequence_length=16, guidance_scale=4.5)
    assert enc["prompt_embeds"].shape == (1, CLIP_TOKENS + 16, 256) and enc["pooled_prompt_embeds"].shape == (1, 64)
    assert enc["negative_prompt_embeds"].shape == enc["prompt_embeds"].shape
    assert not torch.equal(enc["negative_prompt_embeds"], enc["prompt_embeds"])
    with pytest.raises(ValueError, match="pooled_dim"):
        build_sd3_5_runtime_bundle_from_cfg(load_config("experiment/sd3_5_ocr_grpo", overrides=[
            "model.random_init=true", "model.use_lora=false", "model.arch.num_layers=2", "model.arch.hidden_size=64",
            "model.arch.num_heads=2", "model.arch.context_dim=256", "model.arch.pooled_dim=48",
            "model.arch.in_channels=4", f"+model.text_encoder.path={sd3_dir}"]), "cpu", torch.float32)

    wan_cfg = load_config("experiment/wan_2_1_1_3b_grpo", overrides=[
        "model.random_init=true", "model.use_lora=false", "model.dtype=float32", "model.arch.num_layers=2",
        "model.arch.hidden_size=64", "model.arch.num_heads=2", "model.arch.ffn_dim=128", "model.arch.in_channels=4",
        "model.arch.text_dim=32", "model.arch.freq_dim=32", f"+model.text_encoder.path={wan_dir}"])
    wan = build_wan_2_1_runtime_bundle_from_cfg(wan_cfg, "cpu", torch.float32).policy
    assert isinstance(wan.backend_handle.text, UMT5PromptEncoder)
    out = wan.encode_prompt([PROMPT], max_sequence_length=24, guidance_scale=1.0)
    assert out["prompt_embeds"].shape == (1, 24, 32) and out["negative_prompt_embeds"] is None
    assert float(out["prompt_embeds"][0, len(PROMPT) + 1:].abs().max()) == 0.0
