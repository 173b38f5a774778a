"""The sharded-parameter runtime in a single process (world size 1, CPU): one rank is left alone
(no sharding, same outputs, same state dict), and the gather-ahead policy is validated where it is
read.  The multi-rank behaviour is covered by the gloo and GPU workers of ``test_multiprocess.py``."""

import copy

import pytest
import torch

from visionrl_b200.models.nn.mmdit import MMDiT, MMDiTConfig
from visionrl_b200.parallel.fsdp import ShardedParamRuntime, find_units, shard_model
from visionrl_b200.parallel.mesh import ProcessMesh

ARCH = dict(num_layers=2, hidden_size=128, num_heads=2, patch_size=2, in_channels=4, context_dim=64,
            pooled_dim=32, max_grid=8)


def _inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(2, 4, 8, 8, generator=g), torch.rand(2, generator=g) * 1000,
            torch.randn(2, 8, 64, generator=g), torch.randn(2, 32, generator=g))


def _net():
    torch.manual_seed(3)
    return MMDiT(MMDiTConfig(**ARCH)).float()


def test_a_single_rank_is_left_unsharded_and_untouched():
    net = _net()
    ref = copy.deepcopy(net)
    assert len(find_units(net)) == ARCH["num_layers"]                 # the blocks are the gather / reduce units
    rt = shard_model(net, ProcessMesh.build(), torch.device("cpu"), collectives="nccl", ring=2,
                     rollout_replica=True)
    assert rt is None                                                   # nothing to shard over one rank
    x = _inputs()
    assert torch.equal(net(*x), ref(*x))
    assert all(torch.equal(a, b) for a, b in zip(net.state_dict().values(), ref.state_dict().values()))
    assert not any(getattr(m, "sharded", None) is not None for m in net.modules())


def test_gather_ahead_policy_is_validated(monkeypatch):
    for good in ("small", "deep", "all"):
        monkeypatch.setenv("VRL_GATHER_AHEAD", good)
        assert ShardedParamRuntime(ProcessMesh.build(), torch.device("cpu")).forward_ahead == good
    monkeypatch.setenv("VRL_GATHER_AHEAD", "sometimes")
    with pytest.raises(ValueError, match="VRL_GATHER_AHEAD"):
        ShardedParamRuntime(ProcessMesh.build(), torch.device("cpu"))
    monkeypatch.delenv("VRL_GATHER_AHEAD")
    assert ShardedParamRuntime(ProcessMesh.build(), torch.device("cpu")).forward_ahead == "deep"
