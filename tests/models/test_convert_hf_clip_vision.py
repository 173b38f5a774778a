"""The reward tower against ``transformers.CLIPVisionModelWithProjection``: converted weights
must give the same image embeddings, for both activations CLIP checkpoints come with, and a
directory in the Hugging Face layout must load through ``build_image_tower`` as it is."""

import json

import pytest
import torch

from visionrl_b200.models import convert
from visionrl_b200.models.nn.vision import ViTScorer
from visionrl_b200.rewards.vision_tower import build_image_tower

transformers = pytest.importorskip("transformers")


def _hf(act, seed=0):
    torch.manual_seed(seed)
    cfg = transformers.CLIPVisionConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                                        num_attention_heads=2, image_size=32, patch_size=8, projection_dim=24,
                                        hidden_act=act)
    return transformers.CLIPVisionModelWithProjection(cfg).eval(), cfg


def _normalised(t):
    return t / t.norm(dim=-1, keepdim=True)


@pytest.mark.parametrize("hf_act,act", [("quick_gelu", "quick_gelu"), ("gelu", "gelu")])
def test_converted_tower_gives_the_same_image_embeddings(hf_act, act):
    hf, _ = _hf(hf_act)
    state = convert.clip_vision_from_hf(hf.state_dict())
    shape = convert.clip_vision_shape(state)
    assert shape == {"layers": 3, "dim": 128, "mlp": 256, "patch": 8, "image": 32, "out_dim": 24}
    tower = ViTScorer(heads=2, act=act, **shape).eval()
    missing = tower.load_state_dict(state, strict=False)
    assert not missing.unexpected_keys and all(k.startswith(("score_head.", "mean", "std")) for k in missing.missing_keys)
    images01 = torch.rand(3, 3, 32, 32)
    pixel_values = (images01 - tower.mean) / tower.std          # the normalisation the tower applies itself
    with torch.no_grad():
        want = _normalised(hf(pixel_values=pixel_values).image_embeds)
        got = tower.features(images01)
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    # the wrong activation is a different function: the check above is not vacuous
    other = ViTScorer(heads=2, act="gelu_tanh" if act != "gelu_tanh" else "gelu", **shape).eval()
    other.load_state_dict(state, strict=False)
    with torch.no_grad():
        assert not torch.allclose(other.features(images01), want, atol=2e-5)


def test_a_hugging_face_directory_loads_as_it_is(tmp_path):
    from safetensors.torch import save_file

    hf, cfg = _hf("quick_gelu", seed=1)
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"vision_config": cfg.to_dict()}))
    tower = build_image_tower(str(tmp_path), "cpu", torch.float32)
    assert tower.act == "quick_gelu" and tower.blocks[0].heads == 2 and not any(p.requires_grad for p in tower.parameters())
    images01 = torch.rand(2, 3, 32, 32)
    with torch.no_grad():
        want = _normalised(hf(pixel_values=(images01 - tower.mean) / tower.std).image_embeds)
    assert torch.allclose(tower.features(images01), want, atol=2e-5)
    # the native file written by the command-line converter loads the same way
    assert convert.main(["clip_vision", str(tmp_path), str(tmp_path / "native")]) == 0
    (tmp_path / "native" / "config.json").write_text(json.dumps({"vision_config": cfg.to_dict()}))
    again = build_image_tower(str(tmp_path / "native"), "cpu", torch.float32)
    assert torch.equal(again.features(images01), tower.features(images01))


def test_what_is_not_a_clip_tower_is_refused(tmp_path):
    with pytest.raises(KeyError, match="no CLIP vision tower"):
        convert.clip_vision_from_hf({"text_model.embeddings.token_embedding.weight": torch.zeros(2, 2)})
    with pytest.raises(FileNotFoundError, match="random_init"):
        build_image_tower(str(tmp_path / "nowhere"), "cpu", torch.float32)
    with pytest.raises(ValueError, match="unknown ViT activation"):
        ViTScorer(layers=1, dim=32, heads=2, mlp=64, patch=8, image=32, out_dim=8, act="relu")
