"""Mixture-of-experts feed-forward path (kernel K12 and its oracle).

Routing: softmax over expert logits, top-``k`` experts per token with renormalised weights;
tokens are permuted expert-major (stable), every expert runs its two-layer MLP on its
contiguous slice with the tcgen05 GEMM, and the results are combined with the gate weights.
The reference has no MoE layer (its only "experts" are the two timestep-specialised Wan
transformers, ``vrl/models/families/wan_2_1/official_policy.py:276-285``); this block is an
optional drop-in for the dense FFN of the DiT blocks.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


def route_reference(logits: torch.Tensor, top_k: int):
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    return w / w.sum(dim=-1, keepdim=True), idx.to(torch.int32)


def permute_reference(experts: torch.Tensor, num_experts: int):
    flat = experts.reshape(-1).to(torch.int64)
    perm = torch.sort(flat, stable=True).indices.to(torch.int32)
    inv = torch.empty_like(perm)
    inv[perm.long()] = torch.arange(perm.numel(), device=perm.device, dtype=torch.int32)
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32, device=experts.device)
    offsets[1:] = counts.cumsum(0).to(torch.int32)
    return perm, inv, offsets


def _kernels(x: torch.Tensor) -> bool:
    from visionrl_b200.ops import _ext

    return x.is_cuda and _ext.kernels_enabled() and _ext.has("moe_gate_topk")


def route(logits: torch.Tensor, top_k: int):
    """``logits[T, E]`` → ``(weights[T, k] fp32, experts[T, k] int32)``."""
    if _kernels(logits) and logits.shape[-1] <= 64 and top_k <= 8:
        from visionrl_b200.ops import _ext

        w, idx = _ext.load().moe_gate_topk(logits.contiguous(), int(top_k))
        return w, idx
    return route_reference(logits, top_k)


def permute(experts: torch.Tensor, num_experts: int):
    if _kernels(experts):
        from visionrl_b200.ops import _ext

        perm, inv, offsets = _ext.load().moe_permute(experts.contiguous().view(-1), int(num_experts))
        return perm, inv, offsets
    return permute_reference(experts, num_experts)


class _GatherRows(torch.autograd.Function):
    """``xp[pos] = x[perm[pos] // k]`` (backward: scatter-add over the k slots)."""

    @staticmethod
    def forward(ctx, x, perm, top_k):
        ctx.save_for_backward(perm)
        ctx.top_k, ctx.tokens = top_k, x.shape[0]
        if _kernels(x) and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
            from visionrl_b200.ops import _ext

            return _ext.load().moe_gather_rows(x.contiguous(), perm, int(top_k))
        return x[(perm.long() // top_k)]

    @staticmethod
    def backward(ctx, g):
        (perm,) = ctx.saved_tensors
        gx = torch.zeros(ctx.tokens, g.shape[1], dtype=torch.float32, device=g.device)
        gx.index_add_(0, perm.long() // ctx.top_k, g.float())
        return gx.to(g.dtype), None, None


class _Combine(torch.autograd.Function):
    """``y[t] = sum_s w[t, s] yp[inv[t, s]]``."""

    @staticmethod
    def forward(ctx, yp, inv, weights):
        ctx.save_for_backward(yp, inv, weights)
        if _kernels(yp) and yp.dtype == torch.bfloat16 and yp.shape[1] % 8 == 0:
            from visionrl_b200.ops import _ext

            return _ext.load().moe_combine(yp.contiguous(), inv.contiguous().view(-1),
                                           weights.contiguous().float())
        rows = yp[inv.long().view(weights.shape)]                  # [T, k, D]
        return (rows.float() * weights.float().unsqueeze(-1)).sum(dim=1).to(yp.dtype)

    @staticmethod
    def backward(ctx, gy):
        yp, inv, weights = ctx.saved_tensors
        idx = inv.long().view(weights.shape)
        g_rows = gy.float().unsqueeze(1) * weights.float().unsqueeze(-1)      # [T, k, D]
        g_yp = torch.zeros_like(yp, dtype=torch.float32)
        g_yp.index_add_(0, idx.reshape(-1), g_rows.reshape(-1, gy.shape[-1]))
        g_w = (yp[idx].float() * gy.float().unsqueeze(1)).sum(dim=-1)
        return g_yp.to(yp.dtype), None, g_w.to(weights.dtype)


class MoEFFN(nn.Module):
    """Top-``k`` routed feed-forward block: ``E`` experts of ``dim → hidden → dim`` (GELU-tanh)."""

    def __init__(self, dim: int, hidden: int, num_experts: int = 8, top_k: int = 2):
        super().__init__()
        self.dim, self.hidden, self.num_experts, self.top_k = dim, hidden, num_experts, top_k
        self.gate = nn.Linear(dim, num_experts, bias=False)
        self.w1 = nn.Parameter(torch.empty(num_experts, hidden, dim))
        self.b1 = nn.Parameter(torch.zeros(num_experts, hidden))
        self.w2 = nn.Parameter(torch.empty(num_experts, dim, hidden))
        self.b2 = nn.Parameter(torch.zeros(num_experts, dim))
        for e in range(num_experts):
            nn.init.xavier_uniform_(self.w1[e])
            nn.init.xavier_uniform_(self.w2[e])

    def _gate_weights(self, logits: torch.Tensor):
        """Kernel routing for the indices; the weights stay differentiable w.r.t. the logits."""
        _, idx = route(logits.detach(), self.top_k)
        probs = torch.softmax(logits.float(), dim=-1)
        w = probs.gather(-1, idx.long())
        return w / w.sum(dim=-1, keepdim=True), idx

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from visionrl_b200.ops.linear import linear

        shape = x.shape
        tokens = x.reshape(-1, shape[-1])
        weights, experts = self._gate_weights(self.gate(tokens))
        perm, inv, offsets = permute(experts, self.num_experts)
        xp = _GatherRows.apply(tokens, perm, self.top_k)
        bounds = offsets.tolist()                     # one host read per layer: slice boundaries
        outs = []
        for e in range(self.num_experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi == lo:
                continue
            h = linear(xp[lo:hi], self.w1[e], self.b1[e], act="gelu_tanh")
            outs.append(linear(h, self.w2[e], self.b2[e]))
        yp = torch.cat(outs, dim=0) if outs else xp.new_zeros(xp.shape)
        y = _Combine.apply(yp, inv, weights.to(torch.float32))
        return y.view(shape)


def moe_ffn_reference(module: MoEFFN, x: torch.Tensor) -> torch.Tensor:
    """Dense per-expert loop in fp32 (the oracle)."""
    tokens = x.reshape(-1, x.shape[-1]).float()
    weights, experts = route_reference(module.gate(tokens.to(x.dtype)).float(), module.top_k)
    out = torch.zeros_like(tokens)
    for e in range(module.num_experts):
        h = F.gelu(tokens @ module.w1[e].float().t() + module.b1[e].float(), approximate="tanh")
        ye = h @ module.w2[e].float().t() + module.b2[e].float()
        mask = (experts == e).float() * weights
        out += ye * mask.sum(dim=-1, keepdim=True)
    return out.view(x.shape).to(x.dtype)


__all__ = ["MoEFFN", "moe_ffn_reference", "permute", "permute_reference", "route", "route_reference"]
