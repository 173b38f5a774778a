"""``vrl.trainers.fsdp`` on one CPU process: what ``fsdp_wrapper`` attaches for each strategy,
the single-file checkpoint, and the optimiser-state offload hooks (reference expectations:
``vrl/trainers/fsdp.py:35-183``)."""

import pytest
import torch
from safetensors.torch import load_file
from torch import nn

from visionrl_b200.trainers.fsdp import (
    FSDPConfig, OptimizerOffloadHook, fsdp_wrapper, init_distributed, register_optimizer_offload_hooks,
    save_fsdp_checkpoint,
)


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b = nn.Linear(8, 16), nn.Linear(16, 4)
        self.checkpointing = None

    def enable_gradient_checkpointing(self, flag=True):
        self.checkpointing = flag

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


def test_config_defaults_follow_the_reference():
    cfg = FSDPConfig()
    assert (cfg.sharding_strategy, cfg.backward_prefetch, cfg.cpu_offload) == ("FULL_SHARD", "BACKWARD_PRE", False)
    assert (cfg.num_replicate, cfg.num_shard, cfg.mixed_precision_dtype) == (1, 8, torch.bfloat16)
    assert cfg.use_activation_checkpointing is False and cfg.use_device_mesh is False


@pytest.mark.parametrize("strategy,shards_optimizer", [("FULL_SHARD", True), ("SHARD_GRAD_OP", True),
                                                       ("HYBRID_SHARD", True), ("NO_SHARD", False)])
def test_wrapper_returns_the_same_module_with_a_gradient_runtime(strategy, shards_optimizer):
    net = _Net()
    out = fsdp_wrapper(net, FSDPConfig(sharding_strategy=strategy, use_activation_checkpointing=True),
                       collectives="nccl")
    assert out is net and net.checkpointing is True
    runtime = net.sharded_runtime
    # a single process has nothing to shard over, whatever the strategy asks for
    assert runtime.shard_optimizer is False and shards_optimizer in (True, False)
    assert getattr(net, "param_runtime", None) is None
    assert callable(runtime.reduce_clip_step) and callable(runtime.prepare)


def test_wrapper_reaches_an_inner_transformer_for_activation_checkpointing():
    class Policy(nn.Module):
        def __init__(self):
            super().__init__()
            self.transformer = _Net()

    policy = Policy()
    fsdp_wrapper(policy, FSDPConfig(sharding_strategy="NO_SHARD", use_activation_checkpointing=True))
    assert policy.transformer.checkpointing is True


def test_sharding_units_follow_the_layer_classes_and_skip_ignored_modules():
    from visionrl_b200.trainers.fsdp import sharding_units

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(4, 4)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList(Block() for _ in range(3))
            self.frozen = nn.ModuleList(Block() for _ in range(2))

    model = Model()
    assert sharding_units(model) is None                                   # the model's own block list
    assert len(sharding_units(model, lambda: [Block])) == 5
    kept = sharding_units(model, lambda: [Block], ignored_modules=[model.frozen])
    assert len(kept) == 3 and all(any(k is b for b in model.blocks) for k in kept)
    assert len(sharding_units(model, None, ignored_modules=[model.blocks[0]])) == 2
    # the reference's positional call shape
    assert fsdp_wrapper(model, FSDPConfig(sharding_strategy="NO_SHARD"), lambda: [Block], [model.frozen]) is model


def test_single_file_checkpoint_round_trips(tmp_path):
    net = _Net()
    path = save_fsdp_checkpoint(str(tmp_path), net, 7)
    assert path.endswith("checkpoint-7")
    state = load_file(f"{path}/model.safetensors")
    assert set(state) == set(net.state_dict()) and all(torch.equal(state[k], v) for k, v in net.state_dict().items())
    # any other rank writes nothing
    other = save_fsdp_checkpoint(str(tmp_path), net, 8, 1)
    assert not (tmp_path / "checkpoint-8").exists() and other.endswith("checkpoint-8")


def test_offload_hooks_park_the_state_on_the_host_around_every_step():
    torch.manual_seed(0)
    net, twin = _Net(), _Net()
    twin.load_state_dict(net.state_dict())
    opt, twin_opt = torch.optim.AdamW(net.parameters(), lr=1e-2), torch.optim.AdamW(twin.parameters(), lr=1e-2)

    def step(x):
        for model, optimiser in ((net, opt), (twin, twin_opt)):
            optimiser.zero_grad()
            model(x).sum().backward()
            optimiser.step()

    step(torch.randn(3, 8))
    handles, hook = register_optimizer_offload_hooks(opt)
    assert len(handles) == 2 and isinstance(hook, OptimizerOffloadHook)
    weight = net.a.weight
    # between steps the moments live in the hook's host copies and the optimiser holds placeholders
    assert opt.state[weight]["exp_avg"].numel() == 0 and hook.cpu_states[weight]["exp_avg"].shape == weight.shape
    assert opt.state[weight]["step"].numel() == 1                     # the step counter stays where it is
    step(torch.randn(3, 8))
    step(torch.randn(3, 8))
    # every step saw the full state: bit for bit the run without offloading
    assert all(torch.equal(a, b) for a, b in zip(net.parameters(), twin.parameters()))
    assert opt.state[weight]["exp_avg"].numel() == 0 and weight in hook.cpu_states
    assert torch.equal(hook.cpu_states[weight]["exp_avg"], twin_opt.state[twin.a.weight]["exp_avg"])
    for h in handles:
        h.remove()


def test_init_distributed_without_a_launcher_is_a_single_rank(monkeypatch):
    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(name, raising=False)
    assert init_distributed() == (False, 0, 1, 0)
