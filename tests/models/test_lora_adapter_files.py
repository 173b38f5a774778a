"""The adapter export of a checkpoint's ``lora_weights/`` directory: what is written, that it
loads back bit for bit into a freshly adapted network, what a mismatching file is refused for,
and the two ways of getting the base model out of an adapted one."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from visionrl_b200.models.nn import layers as L


class _Net(L.AdapterMixin, torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.qkv = L.LoRALinear(16, 48)
        self.out = L.LoRALinear(16, 16)
        self.plain = L.Linear(16, 16)

    def forward(self, x):
        return self.plain(self.out(self.qkv(x)[..., :16]))


def _adapted(seed):
    torch.manual_seed(seed)
    net = _Net()
    L.apply_lora(net, 4, 8.0, ["qkv", "out"])
    with torch.no_grad():
        for m in L.iter_lora_layers(net):
            m.lora_B.normal_(std=0.1)
    return net


def test_export_writes_both_files_and_loads_back_bit_for_bit(tmp_path):
    src = _adapted(0)
    config = src.save_pretrained(tmp_path / "lora_weights")
    assert config == json.loads((tmp_path / "lora_weights" / L.ADAPTER_CONFIG_NAME).read_text())
    assert config["r"] == 4 and config["lora_alpha"] == 8.0 and config["target_modules"] == ["qkv", "out"]
    stored = load_file(tmp_path / "lora_weights" / L.ADAPTER_WEIGHTS_NAME)
    assert sorted(stored) == ["out.lora_A", "out.lora_B", "qkv.lora_A", "qkv.lora_B"]
    assert stored["qkv.lora_A"].shape == (4, 16) and stored["qkv.lora_B"].shape == (48, 4)

    dst = _adapted(1)
    dst.plain.load_state_dict(src.plain.state_dict())
    for a, b in ((dst.qkv, src.qkv), (dst.out, src.out)):
        a.weight.data.copy_(b.weight.data)
        a.bias.data.copy_(b.bias.data)
    x = torch.randn(3, 16)
    assert not torch.equal(dst(x), src(x))
    assert dst.load_adapter(tmp_path / "lora_weights") == sorted(stored)
    assert torch.equal(dst(x), src(x))


def test_files_that_do_not_fit_the_model_are_refused(tmp_path):
    net = _adapted(0)
    net.save_pretrained(tmp_path / "ok")
    state = load_file(tmp_path / "ok" / L.ADAPTER_WEIGHTS_NAME)

    def write(name, tensors):
        (tmp_path / name).mkdir()
        save_file(tensors, tmp_path / name / L.ADAPTER_WEIGHTS_NAME)
        return tmp_path / name

    with pytest.raises(ValueError, match="unexpected LoRA keys"):
        net.load_adapter(write("extra", {**state, "ghost.lora_A": torch.zeros(4, 16)}))
    with pytest.raises(ValueError, match="lacks LoRA keys"):
        net.load_adapter(write("short", {k: v for k, v in state.items() if not k.startswith("out.")}))
    with pytest.raises(ValueError, match="file has"):
        net.load_adapter(write("rank8", {**state, "qkv.lora_A": torch.zeros(8, 16)}))
    with pytest.raises(RuntimeError, match="without LoRA adapters"):
        _Net().save_pretrained(tmp_path / "none")


def test_zeroed_adapters_give_the_base_model_and_come_back():
    net = _adapted(0)
    x = torch.randn(5, 16)
    with torch.no_grad():
        tuned = net(x)
        with net.disable_adapter():
            base = net(x)
        before = [m.lora_B.clone() for m in L.iter_lora_layers(net)]
        with L.adapters_zeroed(net):
            assert torch.equal(net(x), base)
            # what a weight push would carry inside the block is the base model too
            assert all(float(v.abs().sum()) == 0.0 for k, v in L.lora_state_dict(net).items() if k.endswith("lora_B"))
        assert torch.equal(net(x), tuned) and not torch.equal(tuned, base)
    assert all(torch.equal(m.lora_B, b) for m, b in zip(L.iter_lora_layers(net), before))
    with pytest.raises(RuntimeError):
        with L.adapters_zeroed(_Net()):
            pass
