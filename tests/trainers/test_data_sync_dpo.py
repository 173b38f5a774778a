"""Prompt data, weight syncers, EMA and the offline DPO trainer (reference expectations:
``tests/trainers/test_data.py``, ``test_weight_sync.py``, ``test_offline_dpo_timesteps.py``)."""

import asyncio
from types import SimpleNamespace

import pytest
import torch
from torch import nn

from visionrl_b200.trainers.data import (DistributedKRepeatSampler, TextPromptDataset,
                                         load_prompt_manifest)
from visionrl_b200.trainers.ema import EMAModuleWrapper
from visionrl_b200.trainers.offline_dpo import (OfflineDPOTrainer, OfflineDPOTrainerConfig,
                                                wan_forward)
from visionrl_b200.trainers.pickapic import LatentPreferenceBatch, PreferenceBatch
from visionrl_b200.trainers.weight_sync import (InMemoryWeightSyncer, RayRuntimeWeightSyncer,
                                                build_runtime_weight_syncer)


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


# ------------------------------------------------------------------------------------ data
def test_two_sampler_ranks_hold_complete_groups(tmp_path):
    path = tmp_path / "prompts.txt"
    path.write_text("\n".join(f'a sign that says "word{i}"' for i in range(40)))
    ds = TextPromptDataset(str(path))
    k, bs, world = 4, 6, 2
    samplers = [DistributedKRepeatSampler(ds, bs, k, world, r, seed=7) for r in range(world)]
    batches = [next(iter(s)) for s in samplers]
    merged = batches[0] + batches[1]
    assert len(merged) == world * bs
    counts = {i: merged.count(i) for i in set(merged)}
    assert len(counts) == world * bs // k and set(counts.values()) == {k}
    samplers[0].set_epoch(1)
    assert next(iter(samplers[0])) != batches[0]
    with pytest.raises(AssertionError):
        DistributedKRepeatSampler(ds, 5, 4, 1, 0)


def test_manifests_txt_quotes_jsonl_and_synthetic(tmp_path):
    txt = tmp_path / "p.txt"
    txt.write_text('a poster with "HELLO WORLD" on it\nno quotes here\n\n')
    ex = load_prompt_manifest(txt)
    assert [e.target_text for e in ex] == ["HELLO WORLD", ""]
    jl = tmp_path / "p.jsonl"
    jl.write_text('{"prompt": "x", "target_text": "T", "task_type": "ocr", "metadata": {"a": 1}}\n')
    (e,) = load_prompt_manifest(jl)
    assert (e.prompt, e.target_text, e.task_type, e.metadata) == ("x", "T", "ocr", {"a": 1})
    syn = load_prompt_manifest("synthetic:5:3")
    assert len(syn) == 5 and syn == load_prompt_manifest("synthetic:5:3")


# ------------------------------------------------------------------------------ weight sync
class _Runtime:
    def __init__(self, with_sync=True):
        self.weight_sync = object() if with_sync else None
        self.updates = []

    async def update_weights(self, state, policy_version):
        self.updates.append((state, policy_version))


def test_runtime_syncer_sends_cpu_tensors_with_increasing_versions():
    rt = _Runtime()
    syncer = build_runtime_weight_syncer(rt)
    assert isinstance(syncer, RayRuntimeWeightSyncer)
    _run(syncer.push({"w": torch.ones(2)}))
    _run(syncer.push({"w": torch.zeros(2)}))
    assert [v for _, v in rt.updates] == [1, 2]
    assert all(t.device.type == "cpu" for s, _ in rt.updates for t in s.values())
    resumed = build_runtime_weight_syncer(_Runtime(), initial_policy_version=7)
    _run(resumed.push({"w": torch.ones(1)}))
    assert resumed._runtime.updates[0][1] == 8 if hasattr(resumed, "_runtime") else True


def test_syncer_only_built_when_runtime_supports_it():
    assert build_runtime_weight_syncer(_Runtime(with_sync=False)) is None
    assert build_runtime_weight_syncer(SimpleNamespace()) is None
    mem = InMemoryWeightSyncer()
    _run(mem.push({"a": torch.ones(1)}))
    assert torch.equal(_run(mem.pull())["a"], torch.ones(1))


# --------------------------------------------------------------------------------------- EMA
def test_ema_warmup_decay_swap_and_state():
    p = nn.Parameter(torch.zeros(3))
    ema = EMAModuleWrapper([p], decay=0.99, update_step_interval=1)
    assert ema.get_current_decay(0) == pytest.approx(0.1)
    assert ema.get_current_decay(10 ** 6) == pytest.approx(0.99)
    with torch.no_grad():
        p.fill_(1.0)
    ema.step([p], 0)
    shadow = ema.state_dict()["ema_parameters"][0]
    assert torch.allclose(shadow, torch.full((3,), 0.9))
    ema.copy_ema_to([p], store_temp=True)
    assert torch.allclose(p.detach(), torch.full((3,), 0.9))
    ema.copy_temp_to([p])
    assert torch.allclose(p.detach(), torch.ones(3))
    other = EMAModuleWrapper([nn.Parameter(torch.zeros(3))], decay=0.5)
    other.load_state_dict(ema.state_dict())
    assert other.state_dict()["decay"] == 0.99


# --------------------------------------------------------------------------------------- DPO
class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.transformer = nn.Conv2d(4, 4, 1)

    def forward(self, x, t, ctx):
        return self.transformer(x)


def _dpo(scheduler, **cfg):
    torch.manual_seed(0)
    policy, ref = _Net(), _Net()
    ref.load_state_dict(policy.state_dict())
    fwd = lambda m, x, t, c, extra=None: m(x, t, c)            # noqa: E731
    return OfflineDPOTrainer(policy, ref, fwd, scheduler, encode_pixels=lambda x: x,
                             encode_text=lambda caps: torch.zeros(len(caps), 2, 8),
                             config=OfflineDPOTrainerConfig(lr=1e-3, mixed_precision="no", **cfg),
                             device="cpu")


def _batch(b=2):
    g = torch.Generator().manual_seed(1)
    return LatentPreferenceBatch(torch.randn(b, 4, 8, 8, generator=g), torch.randn(b, 4, 8, 8, generator=g),
                                 ["c"] * b)


def test_missing_timesteps_raise_and_subset_wins():
    empty = SimpleNamespace(timesteps=torch.tensor([]), sigmas=None)
    with pytest.raises(RuntimeError):
        _dpo(empty)._sample_timesteps(4)
    with pytest.raises(RuntimeError):
        _dpo(SimpleNamespace())._sample_timesteps(4)
    idx = _dpo(empty, timestep_subset=(3, 5))._sample_timesteps(64)
    assert set(idx.tolist()) <= {3, 4}


def test_schedule_entries_are_used_not_raw_indices():
    sched = SimpleNamespace(timesteps=torch.tensor([900.0, 500.0, 100.0]),
                            sigmas=torch.tensor([0.9, 0.5, 0.1, 0.0]))
    tr = _dpo(sched)
    lat, noise = torch.ones(3, 4, 2, 2), torch.zeros(3, 4, 2, 2)
    noisy, target, t_vals = tr._inject_noise(lat, noise, torch.tensor([0, 1, 2]))
    assert t_vals.tolist() == [900.0, 500.0, 100.0]
    assert torch.allclose(noisy[:, 0, 0, 0], torch.tensor([0.1, 0.5, 0.9]))
    assert torch.equal(target, noise - lat)


def test_dpo_step_metrics_and_state_round_trip():
    sched = SimpleNamespace(timesteps=torch.linspace(999, 1, 10), sigmas=torch.linspace(1, 0, 11))
    tr = _dpo(sched, beta=10.0)
    m = tr.step(_batch())
    assert m.loss == pytest.approx(0.6931, abs=1e-3) and m.implicit_acc == 0.0   # policy == reference
    assert tr.global_step == 1
    state = tr.state_dict()
    assert set(state) == {"global_step", "optimizer"}
    other = _dpo(sched)
    other.load_state_dict(state)
    assert other.global_step == 1
    with pytest.raises(TypeError):
        other.load_state_dict([1])


def test_wan_forward_unwraps_transformer_and_preference_batch_layout():
    calls = {}

    class _T(nn.Module):
        def forward(self, hidden_states=None, timestep=None, encoder_hidden_states=None, **kw):
            calls["args"] = (hidden_states.shape, timestep.shape)
            return (hidden_states * 2,)

    policy = SimpleNamespace(transformer=_T())
    out = wan_forward(policy, torch.ones(2, 4, 1, 2, 2), torch.tensor([1.0, 2.0]), torch.zeros(2, 3, 8))
    assert torch.equal(out, torch.full((2, 4, 1, 2, 2), 2.0)) and "args" in calls
    pb = PreferenceBatch(torch.arange(2 * 6 * 1 * 1, dtype=torch.float32).view(2, 6, 1, 1), ["a", "b"])
    stacked = pb.stacked_winner_then_loser()
    assert stacked.shape == (4, 3, 1, 1) and stacked[0, :, 0, 0].tolist() == [0.0, 1.0, 2.0]
    assert stacked[2, :, 0, 0].tolist() == [3.0, 4.0, 5.0]
