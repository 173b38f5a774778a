"""Mixture-of-experts feed-forward path (kernel K12 and its oracle).

Routing: softmax over expert logits, top-``k`` experts per token with renormalised weights;
tokens are permuted expert-major (stable) into a row space padded to the GEMM tile height, both
expert layers run as ONE grouped tcgen05 launch each, scheduled from a device-side tile table
(no routing count is read on the host), and the results are combined with the gate weights.
Without the extension the experts run one after another on their slices.
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

        perm, inv, offsets, _ = _ext.load().moe_permute(experts.contiguous().view(-1), int(num_experts), 1)
        return perm, inv, offsets
    return permute_reference(experts, num_experts)


TILE_ROWS = 128          # tile height of the grouped product: every expert's run is padded to it


def permute_padded(experts: torch.Tensor, num_experts: int):
    """Expert-major permutation into a row space where every expert's run starts on a multiple of
    :data:`TILE_ROWS`.  Returns ``(perm, inv, offsets, tile_expert)``: ``perm`` has one entry per
    padded row (-1 in the padding), ``offsets`` the padded starts, ``tile_expert`` the expert of
    every tile (-1 past the last).  All sizes depend on the token count only, so nothing is read
    back to the host."""
    from visionrl_b200.ops import _ext

    return tuple(_ext.load().moe_permute(experts.contiguous().view(-1), int(num_experts), TILE_ROWS))


def permute_padded_reference(experts: torch.Tensor, num_experts: int, pad: int = TILE_ROWS):
    flat = experts.reshape(-1).to(torch.int64)
    n = flat.numel()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + pad - 1) // pad * pad
    starts = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    starts[1:] = padded.cumsum(0)
    slots = ((n + pad - 1) // pad + num_experts) * pad
    perm = torch.full((slots,), -1, dtype=torch.int32, device=flat.device)
    dense_start = torch.zeros(num_experts, dtype=torch.int64, device=flat.device)
    dense_start[1:] = counts.cumsum(0)[:-1]
    e_sorted = flat[order]
    pos = starts[e_sorted] + (torch.arange(n, device=flat.device) - dense_start[e_sorted])
    perm[pos] = order.to(torch.int32)
    inv = torch.empty(n, dtype=torch.int32, device=flat.device)
    inv[order] = pos.to(torch.int32)
    tile_expert = torch.full((slots // pad,), -1, dtype=torch.int32, device=flat.device)
    for e in range(num_experts):
        tile_expert[int(starts[e]) // pad:int(starts[e + 1]) // pad] = e
    return perm, inv, starts.to(torch.int32), tile_expert


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


class _GroupedExpertsFn(torch.autograd.Function):
    """Both expert layers over the padded, expert-sorted rows, each as ONE grouped tcgen05 launch
    scheduled from the device-side tile table: ``y = gelu(xp W1_e^T + b1_e) W2_e^T + b2_e``.

    Backward: ``d(pre)`` comes out of the input-gradient product's gelu-gradient epilogue, the
    weight gradients are grouped products contracting over every expert's row range, the bias
    gradients are per-expert column sums.  No routing count ever reaches the host.
    """

    @staticmethod
    def forward(ctx, xp, w1, b1, w2, b2, offsets, tile_expert):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        h, pre = ext.gemm_grouped(xp, w1, tile_expert, b1, None, 1, False, True)
        y = ext.gemm_grouped(h, w2, tile_expert, b2, None, 0, False, False)[0]
        ctx.save_for_backward(xp, w1, w2, h, pre, offsets, tile_expert)
        return y

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        xp, w1, w2, h, pre, offsets, tile_expert = ctx.saved_tensors
        experts = w1.shape[0]
        gy = gy.contiguous()
        # rows of padding carry garbage forward values; their gradient rows are zero by construction
        # (the combine's backward writes zeros there), which keeps them out of every sum below
        g_pre = ext.gemm_grouped(gy, w2, tile_expert, None, pre, 3, True, False)[0]
        gw2 = ext.gemm_grouped_wgrad(gy, h, offsets, experts)
        gb2 = ext.moe_segment_colsum(gy, offsets, experts)
        gxp = ext.gemm_grouped(g_pre, w1, tile_expert, None, None, 0, True, False)[0]
        gw1 = ext.gemm_grouped_wgrad(g_pre, xp, offsets, experts)
        gb1 = ext.moe_segment_colsum(g_pre, offsets, experts)
        return gxp, gw1, gb1.to(w1.dtype), gw2, gb2.to(w2.dtype), None, None


class _GatherRowsPadded(torch.autograd.Function):
    """``xp[pos] = x[perm[pos] // k]`` into the padded row space (zero rows in the padding)."""

    @staticmethod
    def forward(ctx, x, perm, inv, top_k):
        from visionrl_b200.ops import _ext

        ctx.save_for_backward(inv)
        ctx.top_k = top_k
        return _ext.load().moe_gather_rows(x.contiguous(), perm, int(top_k))

    @staticmethod
    def backward(ctx, g):
        from visionrl_b200.ops import _ext

        (inv,) = ctx.saved_tensors
        # every token reads its k rows back: the combine kernel with unit weights
        ones = torch.ones(inv.numel() // ctx.top_k, ctx.top_k, device=g.device, dtype=torch.float32)
        return _ext.load().moe_combine(g.contiguous(), inv, ones), None, None, None


class _CombinePadded(torch.autograd.Function):
    """``y[t] = sum_s w[t, s] yp[inv[t, s]]`` with kernel backward for both operands."""

    @staticmethod
    def forward(ctx, yp, perm, inv, weights):
        from visionrl_b200.ops import _ext

        ctx.save_for_backward(yp, perm, inv, weights)
        return _ext.load().moe_combine(yp.contiguous(), inv, weights.contiguous())

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        yp, perm, inv, weights = ctx.saved_tensors
        g_yp, g_w = _ext.load().moe_combine_bwd(gy.contiguous(), yp, perm, inv, weights)
        return g_yp, None, None, g_w


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

    def _grouped_ok(self, tokens: torch.Tensor) -> bool:
        """The grouped tcgen05 path: bf16 on CUDA, widths the tile shapes accept."""
        from visionrl_b200.ops import _ext

        return (_kernels(tokens) and tokens.dtype == torch.bfloat16 and self.w1.dtype == torch.bfloat16
                and self.dim % 32 == 0 and self.hidden % 32 == 0 and _ext.has("gemm_grouped")
                and tokens.shape[0] > 0)

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
        if self._grouped_ok(tokens):
            perm, inv, offsets, tile_expert = permute_padded(experts, self.num_experts)
            xp = _GatherRowsPadded.apply(tokens, perm, inv, self.top_k)
            yp = _GroupedExpertsFn.apply(xp, self.w1, self.b1, self.w2, self.b2, offsets, tile_expert)
            y = _CombinePadded.apply(yp, perm, inv.view(-1), weights.to(torch.float32))
            return y.view(shape)
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


__all__ = ["MoEFFN", "TILE_ROWS", "moe_ffn_reference", "permute", "permute_padded", "permute_padded_reference",
           "permute_reference", "route", "route_reference"]
