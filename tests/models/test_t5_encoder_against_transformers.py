"""The native T5 / UMT5 encoder against ``transformers`` on converted weights: shared and
per-layer position bias, gated and plain feed-forward, with and without padding."""

import pytest
import torch

from visionrl_b200.models import convert
from visionrl_b200.models.nn.text_encoders import T5Encoder, T5EncoderConfig, relative_position_bucket

transformers = pytest.importorskip("transformers")

COMMON = dict(vocab_size=80, d_model=48, d_kv=8, d_ff=96, num_layers=3, num_heads=4,
              relative_attention_num_buckets=8, relative_attention_max_distance=12, dropout_rate=0.0)


def _pair(kind, proj):
    torch.manual_seed(0)
    if kind == "umt5":
        cfg = transformers.UMT5Config(feed_forward_proj=proj, **COMMON)
        hf = transformers.UMT5EncoderModel(cfg)
    else:
        cfg = transformers.T5Config(feed_forward_proj=proj, **COMMON)
        hf = transformers.T5EncoderModel(cfg)
    hf = hf.eval()
    with torch.no_grad():                                   # HF initialises the bias tables small; make them matter
        for name, p in hf.named_parameters():
            if "relative_attention_bias" in name:
                p.normal_(std=1.0)
    native_cfg = T5EncoderConfig.from_hf(cfg.to_dict())
    native = T5Encoder(native_cfg).eval()
    native.load_state_dict(convert.t5_encoder_from_hf(hf.state_dict()), strict=True)
    return hf, native, native_cfg


@pytest.mark.parametrize("kind,proj", [("t5", "gated-gelu"), ("umt5", "gated-gelu"), ("t5", "relu")])
def test_hidden_states_agree_with_and_without_padding(kind, proj):
    hf, native, cfg = _pair(kind, proj)
    assert cfg.per_layer_bias is (kind == "umt5") and cfg.gated is proj.startswith("gated")
    ids = torch.randint(0, 80, (2, 20))                     # longer than max_distance: the log buckets are used
    mask = torch.ones(2, 20, dtype=torch.long)
    mask[1, 13:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state
        got = native(ids)
        assert torch.allclose(got, want, atol=3e-5), float((got - want).abs().max())
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got = native(ids, mask)
    assert torch.allclose(got[0], want[0], atol=3e-5)
    assert torch.allclose(got[1, :13], want[1, :13], atol=3e-5)   # padded positions carry no meaning


def test_bias_tables_are_where_the_variant_puts_them():
    _, t5, _ = _pair("t5", "gated-gelu")
    _, umt5, _ = _pair("umt5", "gated-gelu")
    assert [b.rel_bias is not None for b in t5.blocks] == [True, False, False]
    assert all(b.rel_bias is not None for b in umt5.blocks)


def test_bucketing_is_signed_exact_near_zero_and_saturates():
    rel = torch.tensor([-40, -12, -3, -1, 0, 1, 3, 12, 40])
    b = relative_position_bucket(rel, 8, 12)
    assert b.tolist()[4] == 0 and b[3] == 1 and b[5] == 5            # one step back / forward
    assert b[0] == b[1] == 3 and b[7] == b[8] == 7                   # at and beyond the maximum distance
    assert int(b.max()) < 8 and int(b.min()) >= 0


def test_what_is_not_a_t5_encoder_is_refused():
    with pytest.raises(KeyError, match="no T5 encoder"):
        convert.t5_encoder_from_hf({"shared.weight": torch.zeros(2, 2)})
