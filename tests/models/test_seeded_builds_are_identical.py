"""Random-init builds are a function of ``model.init_seed`` alone.  A rollout worker builds its
own copy of the policy and receives only the trainable state from the trainer, so two builds in
one process — with the global generator in different states — must agree bit for bit, frozen
decoder included; otherwise the first replay does not reproduce the rollout's log-probabilities."""

import pytest
import torch

from visionrl_b200.config.loader import load_config

VIDEO = ["model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
         "model.arch.ffn_dim=128", "model.arch.text_dim=32", "model.arch.freq_dim=32", "sampling.num_frames=5",
         "sampling.height=32", "sampling.width=32", "sampling.max_sequence_length=8", "sampling.num_steps=3"]


def _sd3(cfg_overrides=()):
    from visionrl_b200.models.families.sd3_5.builder import build_sd3_5_runtime_bundle_from_cfg

    cfg = load_config("experiment/sd3_5_ocr_grpo", overrides=[
        "model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
        "model.arch.context_dim=32", "model.arch.pooled_dim=32", "model.arch.in_channels=4", "sampling.height=32",
        "sampling.width=32", "sampling.max_sequence_length=8", *cfg_overrides])
    return build_sd3_5_runtime_bundle_from_cfg(cfg, "cpu", torch.float32).policy


def _wan():
    from visionrl_b200.models.families.wan_2_1.builder import build_wan_2_1_runtime_bundle_from_cfg

    cfg = load_config("experiment/wan_2_1_1_3b_grpo", overrides=VIDEO + ["model.arch.in_channels=4"])
    return build_wan_2_1_runtime_bundle_from_cfg(cfg, "cpu", torch.float32).policy


def _cosmos():
    from visionrl_b200.models.families.cosmos.builder import build_cosmos_predict2_runtime_bundle_from_cfg

    cfg = load_config("experiment/cosmos_predict2_2b_grpo", overrides=VIDEO)
    return build_cosmos_predict2_runtime_bundle_from_cfg(cfg, "cpu", torch.float32).policy


def _janus():
    from visionrl_b200.models.families.janus_pro.policy import JanusProConfig, JanusProPolicy

    arch = {"num_layers": 2, "hidden_size": 64, "num_heads": 2, "ffn_dim": 128, "vocab_size": 128,
            "image_vocab_size": 96, "codebook_dim": 8, "vq_base": 16, "vq_mults": [1, 2], "vq_blocks": 1}
    return JanusProPolicy(JanusProConfig(arch=arch, random_init=True, dtype="float32", use_lora=False,
                                         image_token_num=9, image_size=32))


def _nextstep():
    from visionrl_b200.models.families.nextstep_1.policy import NextStep1Config, NextStep1Policy

    arch = {"num_layers": 2, "hidden_size": 64, "num_heads": 2, "ffn_dim": 128, "vocab_size": 128, "token_dim": 16,
            "head_hidden": 32, "head_layers": 2, "token_patch": 2, "vae_base": 8, "vae_mults": [1, 2], "vae_blocks": 1}
    return NextStep1Policy(NextStep1Config(arch=arch, random_init=True, dtype="float32", use_lora=False))


def _all_tensors(policy):
    """Trainable network and the frozen decoders, which are plain attributes outside ``state_dict``."""
    # (adapter factors are drawn afterwards and reach a worker through the weight push)
    out = {f"net.{k}": v for k, v in policy.state_dict().items() if "lora_" not in k}
    for name in ("_vq", "_vae"):
        frozen = policy.__dict__.get(name)
        if frozen is not None:
            out.update({f"{name}.{k}": v for k, v in frozen.state_dict().items()})
    handle = getattr(policy, "backend_handle", None)
    decoder = getattr(handle, "decoder", None)
    if decoder is not None:
        out.update({f"decoder.{k}": v for k, v in decoder.state_dict().items()})
    return out


@pytest.mark.parametrize("build", [_sd3, _wan, _cosmos, _janus, _nextstep])
def test_two_builds_agree_whatever_was_drawn_before(build):
    torch.manual_seed(1)
    first = _all_tensors(build())
    torch.manual_seed(2)
    torch.randn(17)                                   # the global generator has moved on
    second = _all_tensors(build())
    assert first.keys() == second.keys() and len(first) > 10
    worst = max(float((first[k].float() - second[k].float()).abs().max()) for k in first)
    assert worst == 0.0
    assert any(k.startswith(("decoder.", "_vq.", "_vae.")) for k in first)


def test_another_seed_gives_other_weights():
    a, b = _all_tensors(_sd3()), _all_tensors(_sd3(["+model.init_seed=5"]))
    assert any(not torch.equal(a[k], b[k]) for k in a if k.startswith("net."))
