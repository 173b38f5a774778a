"""The trainer-facing contract every diffusion policy inherits from ``DiffusionPolicy``: it is an
``nn.Module`` whose one trainable child is the transformer, ``forward`` is the denoising step,
replay rebuilds the step's state from a batch, the adapter-off context belongs to the transformer,
and weight pushes are ``transformer.``-prefixed payloads that must cover what trains.  Reference
expectations: ``tests/models/test_diffusion_policy_module.py``."""

import contextlib

import pytest
import torch
from torch import nn

from visionrl_b200.models.diffusion import DiffusionPolicy


class _Transformer(nn.Module):
    def __init__(self):
        super().__init__()
        self.base = nn.Linear(3, 3)
        self.adapter = nn.Linear(3, 3, bias=False)
        self.base.requires_grad_(False)
        self.disabled = False

    @contextlib.contextmanager
    def disable_adapter(self):
        self.disabled = True
        try:
            yield
        finally:
            self.disabled = False

    def forward(self, x):
        return self.base(x) + (0 if self.disabled else self.adapter(x))


class _Policy(DiffusionPolicy):
    family = "stub"

    def __init__(self, with_transformer=True):
        super().__init__()
        if with_transformer:
            self.transformer = _Transformer()
        object.__setattr__(self, "frozen_tower", nn.Linear(2, 2))      # a helper that must not register
        self.restored = []

    def encode_prompt(self, prompt, negative_prompt=None, **kwargs):
        return {"prompt": prompt}

    def prepare_sampling(self, request, encoded, **kwargs):
        return {"latents": torch.zeros(1, 3)}

    def forward_step(self, state, step_idx):
        return {"noise_pred": self.transformer(state["latents"]), "step": step_idx}

    def decode_latents(self, latents):
        return latents

    def restore_eval_state(self, batch_extras, batch_context, latents, step_idx):
        self.restored.append(step_idx)
        return {"latents": latents}


class _Batch:
    def __init__(self):
        self.observations = torch.arange(24, dtype=torch.float32).view(2, 4, 3)
        self.extras, self.context = {}, {}


def test_only_the_transformer_is_a_registered_child_and_its_parameters_are_the_policy_s():
    policy = _Policy()
    assert [name for name, _ in policy.named_children()] == ["transformer"]
    assert {n.split(".")[0] for n, _ in policy.named_parameters()} == {"transformer"}
    assert policy.describe() == {"family": "stub"}


def test_calling_the_policy_is_the_denoising_step():
    policy = _Policy()
    state = {"latents": torch.ones(2, 3)}
    out = policy(state, 3)
    assert out["step"] == 3 and torch.equal(out["noise_pred"], policy.forward_step(state, 3)["noise_pred"])


def test_replay_restores_the_step_state_from_the_batch_and_runs_one_forward():
    policy, batch = _Policy(), _Batch()
    out = policy.replay_forward(batch, 2)
    assert policy.restored == [2] and out["step"] == 0                 # eval states are packed for index 0
    assert torch.equal(out["noise_pred"], policy.transformer(batch.observations[:, 2]))
    assert out["noise_pred"].requires_grad                              # gradients reach the adapter


def test_adapter_off_context_is_the_transformer_s_own():
    policy = _Policy()
    x = torch.ones(1, 3)
    with policy.disable_adapter():
        assert policy.transformer.disabled is True
        off = policy(dict(latents=x), 0)["noise_pred"]
    assert policy.transformer.disabled is False
    assert torch.equal(off, policy.transformer.base(x))
    with pytest.raises(RuntimeError, match="no registered trainable transformer"):
        _Policy(with_transformer=False).disable_adapter()
    bare = _Policy()
    bare.transformer = nn.Linear(3, 3)
    with pytest.raises(RuntimeError, match="does not expose disable_adapter"):
        bare.disable_adapter()


def test_weight_push_payload_is_exactly_what_trains_and_loads_back():
    src, dst = _Policy(), _Policy()
    with torch.no_grad():
        src.transformer.adapter.weight.fill_(2.0)
    payload = src.trainable_state_dict()
    assert list(payload) == ["transformer.adapter.weight"]             # the frozen base is not pushed
    dst.load_trainable_state(payload)
    assert torch.equal(dst.transformer.adapter.weight, src.transformer.adapter.weight)
    full = {f"transformer.{k}": v for k, v in src.transformer.state_dict().items()}
    dst.load_trainable_state(full)                                      # a complete state loads strictly
    assert torch.equal(dst.transformer.base.weight, src.transformer.base.weight)


def test_weight_push_refuses_foreign_empty_and_incomplete_payloads():
    policy = _Policy()
    with pytest.raises(ValueError, match="empty state dict"):
        policy.load_trainable_state({})
    with pytest.raises(ValueError, match="policy keys prefixed"):
        policy.load_trainable_state({"unknown": torch.ones(1)})
    with pytest.raises(ValueError, match="does not have"):
        policy.load_trainable_state({"transformer.nope": torch.ones(1)})
    with pytest.raises(ValueError, match="misses trainable keys"):
        policy.load_trainable_state({"transformer.base.bias": torch.zeros(3)})
