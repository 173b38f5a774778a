"""The native LLaMA decoder against the ``transformers`` implementation: a Hugging Face state
dict goes through the converter (fused projections, rotary row order, names) and both models must
produce the same hidden states — full sequence, with padding, and token by token through the
key/value cache."""

import pytest
import torch

from visionrl_b200.models import convert
from visionrl_b200.models.nn.llama import LlamaConfig, LlamaDecoder

transformers = pytest.importorskip("transformers")

HEADS, HIDDEN, FFN, VOCAB, LAYERS = 4, 64, 160, 96, 3


@pytest.fixture(scope="module")
def pair():
    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(
        vocab_size=VOCAB, hidden_size=HIDDEN, intermediate_size=FFN, num_hidden_layers=LAYERS,
        num_attention_heads=HEADS, num_key_value_heads=HEADS, rms_norm_eps=1e-6, rope_theta=10000.0,
        max_position_embeddings=64, attention_bias=False, mlp_bias=False)
    hf = transformers.LlamaModel(hf_cfg).eval()
    native = LlamaDecoder(LlamaConfig(num_layers=LAYERS, hidden_size=HIDDEN, num_heads=HEADS, ffn_dim=FFN,
                                      vocab_size=VOCAB, rope_theta=10000.0, rms_eps=1e-6, max_positions=64)).eval()
    native.load_state_dict(convert.llama_from_hf(hf.state_dict(), HEADS), strict=True)
    return hf, native


def test_full_sequence_hidden_states_agree(pair):
    hf, native = pair
    ids = torch.randint(0, VOCAB, (2, 11))
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state
        got = native(native.embed_tokens(ids))
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())


def test_left_padded_rows_agree_on_their_real_tokens(pair):
    hf, native = pair
    ids = torch.randint(0, VOCAB, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.long)
    mask[1, :3] = 0
    # positions count every slot, padded or not, in the native decoder; tell transformers the same
    pos = torch.arange(9)[None].expand(2, 9)
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask, position_ids=pos).last_hidden_state
        got = native(native.embed_tokens(ids), attention_mask=mask)
    assert torch.allclose(got[0], want[0], atol=2e-5)
    assert torch.allclose(got[1, 3:], want[1, 3:], atol=2e-5)


def test_token_by_token_decoding_through_the_cache_agrees(pair):
    hf, native = pair
    ids = torch.randint(0, VOCAB, (2, 8))
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state
        cache = native.new_cache(2, 16)
        prefix = native(native.embed_tokens(ids[:, :5]), cache=cache)
        assert torch.allclose(prefix, want[:, :5], atol=2e-5)
        for t in range(5, 8):
            step = native.decode_step_at(native.embed_tokens(ids[:, t]), cache, torch.tensor([t]))
            cache.length = t + 1
            assert torch.allclose(step, want[:, t], atol=3e-5), t


def test_rotary_row_permutation_and_refusals():
    w = torch.arange(8.0).view(8, 1)                     # one head of 8 rows: HF order 0..7
    assert convert._interleave_rotary_rows(w, 1).flatten().tolist() == [0, 4, 1, 5, 2, 6, 3, 7]
    two = convert._interleave_rotary_rows(torch.arange(8.0).view(8, 1), 2).flatten().tolist()
    assert two == [0, 2, 1, 3, 4, 6, 5, 7]               # per head, never across heads
    with pytest.raises(KeyError, match="no LLaMA trunk"):
        convert.llama_from_hf({"embed_tokens.weight": torch.zeros(1)}, 2)
    hf = transformers.LlamaModel(transformers.LlamaConfig(
        vocab_size=32, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4,
        num_key_value_heads=2, mlp_bias=True)).state_dict()
    with pytest.raises(ValueError, match="no native counterpart"):
        convert.llama_from_hf(hf, 4)


def test_janus_mapping_covers_the_generation_side_and_loads_strictly(pair, tmp_path):
    from safetensors.torch import load_file, save_file

    from visionrl_b200.models.families.janus_pro.policy import JanusNetwork

    hf, _ = pair
    codebook, code_dim = 40, 8
    state = {f"language_model.model.{k}": v for k, v in hf.state_dict().items()}
    state["language_model.lm_head.weight"] = torch.zeros(VOCAB, HIDDEN)          # dropped
    state["vision_model.patch_embed.weight"] = torch.zeros(4, 4)                 # dropped
    side = {"gen_embed.weight": (codebook, code_dim),
            "gen_aligner.layers.0.weight": (HIDDEN, code_dim), "gen_aligner.layers.0.bias": (HIDDEN,),
            "gen_aligner.layers.2.weight": (HIDDEN, HIDDEN), "gen_aligner.layers.2.bias": (HIDDEN,),
            "gen_head.output_mlp_projector.weight": (HIDDEN, HIDDEN), "gen_head.output_mlp_projector.bias": (HIDDEN,),
            "gen_head.vision_head.weight": (codebook, HIDDEN), "gen_head.vision_head.bias": (codebook,)}
    state.update({k: torch.randn(shape) for k, shape in side.items()})
    src = tmp_path / "hf"
    src.mkdir()
    save_file({k: v.contiguous() for k, v in state.items()}, str(src / "model.safetensors"))
    assert convert.main(["janus", str(src), str(tmp_path / "native"), "--num-heads", str(HEADS)]) == 0
    native = load_file(str(tmp_path / "native" / "janus.safetensors"))
    net = JanusNetwork({"num_layers": LAYERS, "hidden_size": HIDDEN, "num_heads": HEADS, "ffn_dim": FFN,
                        "vocab_size": VOCAB, "image_vocab_size": codebook, "codebook_dim": code_dim})
    net.load_state_dict(native, strict=True)
    assert torch.equal(net.gen_head.fc2.weight, state["gen_head.vision_head.weight"])
    with pytest.raises(KeyError, match="lacks"):
        convert.janus_from_hf({k: v for k, v in state.items() if not k.startswith("gen_head")}, HEADS)


def test_grouped_query_trunk_with_projection_bias_matches_transformers():
    """A Qwen2-style trunk (two key/value heads for four query heads, bias on q / k / v): converted
    weights give the same hidden states, full sequence and token by token through the cache."""
    torch.manual_seed(0)
    hf_cfg = transformers.Qwen2Config(vocab_size=VOCAB, hidden_size=HIDDEN, intermediate_size=FFN,
                                      num_hidden_layers=LAYERS, num_attention_heads=HEADS, num_key_value_heads=2,
                                      rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=64)
    hf = transformers.Qwen2Model(hf_cfg).eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if name.endswith("_proj.bias"):
                p.normal_(std=0.5)                       # zero-initialised by default: make it matter
    native = LlamaDecoder(LlamaConfig(num_layers=LAYERS, hidden_size=HIDDEN, num_heads=HEADS, ffn_dim=FFN,
                                      vocab_size=VOCAB, rope_theta=10000.0, rms_eps=1e-6, max_positions=64,
                                      num_kv_heads=2, qkv_bias=True)).eval()
    state = convert.llama_from_hf(hf.state_dict(), HEADS)
    assert state["layers.0.attn.qkv.weight"].shape == ((HEADS + 2 * 2) * (HIDDEN // HEADS), HIDDEN)
    native.load_state_dict(state, strict=True)
    assert not native.layers[0].attn.plain_layout
    ids = torch.randint(0, VOCAB, (2, 9))
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state
        got = native(native.embed_tokens(ids))
        assert torch.allclose(got, want, atol=3e-5), float((got - want).abs().max())
        cache = native.new_cache(2, 16)
        prefix = native(native.embed_tokens(ids[:, :6]), cache=cache)
        assert torch.allclose(prefix, want[:, :6], atol=3e-5)
        for t in range(6, 9):
            step = native.decode_step_at(native.embed_tokens(ids[:, t]), cache, torch.tensor([t]))
            cache.length = t + 1
            assert torch.allclose(step, want[:, t], atol=5e-5), t
    with pytest.raises(ValueError, match="multiple of num_kv_heads"):
        LlamaDecoder(LlamaConfig(num_layers=1, hidden_size=64, num_heads=4, ffn_dim=64, vocab_size=8, num_kv_heads=3))
