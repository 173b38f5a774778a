"""NextStep flow-head sampling/replay and the Cosmos reference-image hook (reference expectations:
``tests/engine/generation/test_pipeline_nextstep_1.py:521-546``, ``test_pipeline_cosmos.py``)."""

import math

import pytest
import torch
from torch import nn

from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.models.families.cosmos.executor import CosmosPipelineExecutor
from visionrl_b200.models.families.nextstep_1.flow_step import (flow_logprob_at,
                                                                flow_sample_with_logprob,
                                                                gaussian_token_log_prob)


class _Head(nn.Module):
    input_dim = 6

    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.proj = nn.Linear(6 + 4 + 1, 6)

    def forward(self, x, t, cond):
        tt = t.reshape(-1, 1).expand(x.shape[0], 1).to(x.dtype)
        return self.proj(torch.cat([x, cond, tt], dim=-1))


def test_replay_with_saved_noise_reproduces_the_sampled_log_prob():
    head, cond, unc = _Head(), torch.randn(5, 4), torch.randn(5, 4)
    gen = torch.Generator().manual_seed(1)
    res = flow_sample_with_logprob(head, cond, num_flow_steps=8, noise_level=0.7, cfg_uncond=unc,
                                   cfg_scale=2.0, generator=gen)
    assert res.token.shape == (5, 6) and res.log_prob.shape == (5,)
    again = flow_logprob_at(head, cond, res.token, saved_noise=res.initial_noise, num_flow_steps=8,
                            noise_level=0.7, cfg_uncond=unc, cfg_scale=2.0)
    assert torch.allclose(again, res.log_prob, atol=1e-5)
    assert again.requires_grad                                      # gradients reach the head
    std = 0.7 * math.sqrt(1 / 8)
    assert torch.allclose(res.std, torch.full((5,), std))
    # the log-probability is SUMMED over the token dimension
    manual = (-((res.token - res.mean) ** 2).sum(-1) / (2 * std ** 2) - 6 * math.log(std)
              - 3 * math.log(2 * math.pi))
    assert torch.allclose(gaussian_token_log_prob(res.token, res.mean, std), manual, atol=1e-5)
    with pytest.raises(ValueError):
        flow_sample_with_logprob(head, cond, initial_noise=torch.zeros(2, 6))


def test_cosmos_request_reference_image_overrides_the_constructor_image():
    ex = CosmosPipelineExecutor(model=None, reference_image="ctor.png")
    base = dict(request_id="r", family="cosmos", task="v2w", prompts=["p"], samples_per_prompt=1)
    hook = dict(encoded={}, video_request=None, spec=None, chunk=None)
    plain = GenerationRequest(**base)
    assert ex.build_prepare_kwargs(generation_request=plain, **hook) == {"reference_image": "ctor.png"}
    override = GenerationRequest(**base, metadata={"reference_image": "request.png"})
    assert ex.build_prepare_kwargs(generation_request=override, **hook) == {"reference_image": "request.png"}
    assert ex.respect_cfg_flag is False and (ex.family, ex.task) == ("cosmos", "v2w")


def test_mmdit_with_routed_ffn_runs_and_trains():
    from visionrl_b200.models.nn.mmdit import MMDiT, MMDiTConfig
    from visionrl_b200.ops import moe

    torch.manual_seed(0)
    cfg = MMDiTConfig(num_layers=1, hidden_size=64, num_heads=2, in_channels=4, context_dim=32,
                      pooled_dim=16, max_grid=8, moe_experts=4, moe_top_k=2)
    net = MMDiT(cfg)
    assert isinstance(net.blocks[0].mlp_x.ffn, moe.MoEFFN)
    lat, ctx, pooled = torch.randn(2, 4, 8, 8), torch.randn(2, 5, 32), torch.randn(2, 16)
    out = net(lat, torch.tensor([500.0, 200.0]), ctx, pooled)
    assert out.shape == lat.shape
    out.pow(2).mean().backward()
    ffn = net.blocks[0].mlp_x.ffn
    assert ffn.w1.grad is not None and ffn.gate.weight.grad is not None
    # routing invariants of the oracle
    w, idx = moe.route_reference(torch.randn(7, 4), 2)
    assert torch.allclose(w.sum(-1), torch.ones(7)) and idx.shape == (7, 2)
    perm, inv, off = moe.permute_reference(idx, 4)
    assert off[-1].item() == 14 and torch.equal(perm[inv.long()].long(), torch.arange(14))
