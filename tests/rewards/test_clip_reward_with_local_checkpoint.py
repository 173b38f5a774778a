"""CLIP-score with a local Hugging Face checkpoint directory: the native text tower against
``transformers`` on converted weights, and the reward's number against the one computed with
``transformers.CLIPModel`` from the same files (weights, config, byte-level vocabulary)."""

import asyncio
import json

import pytest
import torch

from visionrl_b200.models import convert
from visionrl_b200.models.nn.vision import CLIPTextTower
from visionrl_b200.rewards.clip import CLIPScoreReward
from visionrl_b200.rewards.pickscore import PickScoreReward

transformers = pytest.importorskip("transformers")


def _bytes_to_unicode():
    """The printable stand-ins of the 256 byte values that byte-level BPE vocabularies use."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs, extra = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + extra)
            extra += 1
    return dict(zip(bs, [chr(c) for c in cs]))


def _byte_level_vocab():
    chars = list(_bytes_to_unicode().values())
    tokens = chars + [c + "</w>" for c in chars] + ["<|startoftext|>", "<|endoftext|>"]
    return {t: i for i, t in enumerate(tokens)}


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    from safetensors.torch import save_file

    root = tmp_path_factory.mktemp("clip")
    vocab = _byte_level_vocab()
    (root / "vocab.json").write_text(json.dumps(vocab))
    (root / "merges.txt").write_text("#version: 0.2\n")
    torch.manual_seed(0)
    eos = vocab["<|endoftext|>"]
    cfg = transformers.CLIPConfig(
        text_config=dict(vocab_size=len(vocab), hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=2, max_position_embeddings=24, hidden_act="quick_gelu",
                         bos_token_id=vocab["<|startoftext|>"], eos_token_id=eos, pad_token_id=eos),
        vision_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                           image_size=32, patch_size=8, hidden_act="quick_gelu"),
        projection_dim=32)
    model = transformers.CLIPModel(cfg).eval()
    with torch.no_grad():
        model.logit_scale.fill_(3.0)
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, str(root / "model.safetensors"))
    (root / "config.json").write_text(json.dumps(cfg.to_dict()))
    tokenizer = transformers.CLIPTokenizer.from_pretrained(str(root))
    return root, model, tokenizer


PROMPTS = ["a red fox", "two boats at dusk, oil painting"]


def test_native_text_tower_matches_transformers_on_converted_weights(checkpoint):
    root, model, tokenizer = checkpoint
    state = convert.clip_text_from_hf(model.state_dict())
    shape = convert.clip_text_shape(state)
    assert shape["context"] == 24 and shape["layers"] == 2 and shape["out_dim"] == 32
    tower = CLIPTextTower(heads=2, act="quick_gelu", eos_token_id=tokenizer.eos_token_id, **shape).eval()
    tower.load_state_dict(state, strict=True)
    batch = tokenizer(PROMPTS, padding="max_length", truncation=True, max_length=24, return_tensors="pt")
    with torch.no_grad():
        want = model.get_text_features(**batch)
        want = getattr(want, "pooler_output", want)
        want = want / want.norm(dim=-1, keepdim=True)
        got = tower.features(batch["input_ids"])
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())


def test_reward_from_the_directory_equals_the_transformers_number(checkpoint):
    root, model, tokenizer = checkpoint
    reward = CLIPScoreReward(device="cpu", model_name=str(root))
    images01 = torch.rand(2, 3, 32, 32)
    got = reward.score_tensor_batch(images01, PROMPTS)
    tower = reward._tower
    batch = tokenizer(PROMPTS, padding="max_length", truncation=True, max_length=24, return_tensors="pt")
    with torch.no_grad():
        out = model(pixel_values=(images01 - tower.mean) / tower.std, **batch)
    want = out.logits_per_image.diagonal() / 30.0            # logit_scale * cosine / 30
    assert reward.logit_scale == pytest.approx(float(torch.tensor(3.0).exp()), rel=1e-6)
    assert torch.allclose(got, want, atol=1e-4), (got, want)
    # the preference-score variant divides by 26 instead
    pick = PickScoreReward(device="cpu", model_name=str(root)).score_tensor_batch(images01, PROMPTS)
    assert torch.allclose(pick * 26.0, got * 30.0, atol=1e-4)


def test_without_tokenizer_files_the_seeded_text_side_is_used(checkpoint, tmp_path):
    import shutil

    root, _, _ = checkpoint
    bare = tmp_path / "bare"
    bare.mkdir()
    for name in ("model.safetensors", "config.json"):
        shutil.copy(root / name, bare / name)
    reward = CLIPScoreReward(device="cpu", model_name=str(bare))
    score = reward.score_tensor_batch(torch.rand(1, 3, 32, 32), ["a red fox"])
    assert reward._text_tower is None and reward.logit_scale == 100.0 and bool(torch.isfinite(score).all())
