"""Token log-probabilities (kernel K7 and its oracle).

``token_log_probs(logits, ids, T)`` = ``log_softmax(logits / T)[ids]`` in fp32.
``fused_head_log_probs(hidden, weight, bias, ids, T)`` computes the same quantity
from the pre-head hidden states with the log-sum-exp folded into the head GEMM's epilogue,
so no fp32 logits exist in HBM.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


_CHUNKED_FOLD = False      # tests flip this to compare the two kernel forms


def token_log_probs_reference(logits, ids, temperature: float = 1.0):
    lp = F.log_softmax(logits.float() / temperature, dim=-1)
    return lp.gather(-1, ids.unsqueeze(-1)).squeeze(-1)


class _TokenLogProbFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, ids, temperature):
        from visionrl_b200.ops import _ext

        flat = logits.reshape(-1, logits.shape[-1]).contiguous()
        lp, lse = _ext.load().token_logprob_fwd(flat, ids.reshape(-1).contiguous(),
                                                float(temperature))
        ctx.save_for_backward(flat, ids.reshape(-1), lse)
        ctx.temperature = temperature
        ctx.shape = logits.shape
        return lp.view(ids.shape)

    @staticmethod
    def backward(ctx, g):
        from visionrl_b200.ops import _ext

        flat, ids, lse = ctx.saved_tensors
        grad = _ext.load().token_logprob_bwd(flat, ids, lse, g.reshape(-1).contiguous().float(),
                                             float(ctx.temperature))
        return grad.view(ctx.shape), None, None


def token_log_probs(logits, ids, temperature: float = 1.0):
    from visionrl_b200.ops import _ext

    if (logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32)
            and _ext.kernels_enabled() and _ext.has("token_logprob_fwd")):
        return _TokenLogProbFn.apply(logits, ids, temperature)
    return token_log_probs_reference(logits, ids, temperature)


def fused_head_log_probs_reference(hidden, weight, bias, ids, temperature: float = 1.0,
                                   chunk: int = 4096):
    """Vocabulary-tiled oracle of the fused kernel (exact, differentiable)."""
    h = hidden.reshape(-1, hidden.shape[-1])
    flat_ids = ids.reshape(-1)
    logits = F.linear(h, weight, bias).float() / temperature
    return token_log_probs_reference(logits, flat_ids, 1.0).view(ids.shape)


class _HeadLogProbFn(torch.autograd.Function):
    """Head GEMM with the log-sum-exp folded into its epilogue.

    Forward: ONE tcgen05 GEMM over the whole vocabulary; each epilogue thread holds 64 consecutive
    logits of one row and reduces them to (max, exponential sum, target value), so 8 bytes per row
    and 64 columns reach memory instead of 256 bytes of fp32 logits; a one-thread-per-row kernel
    merges the partials.  Backward: per vocabulary chunk the product is recomputed with an epilogue
    that writes ``g/T (onehot - softmax)`` as bf16 straight away, which feeds the two gradient
    GEMMs.  No fp32 logits exist in memory in either pass.
    """

    @staticmethod
    def forward(ctx, hidden, weight, bias, ids, temperature, chunk):
        from visionrl_b200.ops import _ext

        h = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        flat_ids = ids.reshape(-1).contiguous()
        logp, lse = _ext.load().head_logprob_fwd(h, weight.contiguous(), bias, flat_ids, float(temperature))
        ctx.save_for_backward(h, weight, bias if bias is not None else h.new_zeros(0), flat_ids, lse)
        ctx.has_bias = bias is not None
        ctx.temperature, ctx.chunk = float(temperature), int(chunk)
        ctx.hidden_shape = hidden.shape
        return logp.view(ids.shape)

    @staticmethod
    def backward(ctx, g):
        from visionrl_b200.ops import _ext
        from visionrl_b200.ops.linear import gemm_nn, gemm_tn

        ext = _ext.load()
        h, weight, bias, flat_ids, lse = ctx.saved_tensors
        bias = bias if ctx.has_bias else None
        gflat = g.reshape(-1).contiguous().float()
        vocab = weight.shape[0]
        need_w = ctx.needs_input_grad[1]
        gh = torch.zeros(h.shape, device=h.device, dtype=torch.float32)
        gw = torch.empty_like(weight) if need_w else None
        gb = torch.empty_like(bias) if (bias is not None and ctx.needs_input_grad[2]) else None
        for c0 in range(0, vocab, ctx.chunk):
            c1 = min(vocab, c0 + ctx.chunk)
            dl = ext.head_softmax_grad(h, weight[c0:c1], None if bias is None else bias[c0:c1], flat_ids,
                                       lse, gflat, c0, ctx.temperature)
            gh += gemm_nn(dl, weight[c0:c1]).float()
            if need_w:
                gw[c0:c1] = gemm_tn(dl, h)
            if gb is not None:
                gb[c0:c1] = ext.colsum(dl).to(gb.dtype)
        return gh.to(h.dtype).view(ctx.hidden_shape), gw, gb, None, None, None


class _FusedHeadLogProbFn(torch.autograd.Function):
    """The same quantity with the fold done by a second kernel per vocabulary chunk (kept for
    extension builds without the epilogue form, and as a cross-check of it).

    Forward: for every vocabulary chunk the tcgen05 GEMM writes fp32 logits ``[rows, chunk]``,
    one kernel folds them into the running (max, sum) and picks up the target logit.  Backward
    recomputes each chunk, turns it into ``g/T (onehot - softmax)`` in bf16 and feeds the two
    gradient GEMMs.
    """

    @staticmethod
    def forward(ctx, hidden, weight, bias, ids, temperature, chunk):
        from visionrl_b200.ops import _ext
        from visionrl_b200.ops.linear import gemm_nt

        ext = _ext.load()
        h = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        flat_ids = ids.reshape(-1).contiguous()
        rows, vocab = h.shape[0], weight.shape[0]
        run_max = torch.full((rows,), float("-inf"), device=h.device, dtype=torch.float32)
        run_sum = torch.zeros(rows, device=h.device, dtype=torch.float32)
        target = torch.zeros(rows, device=h.device, dtype=torch.float32)
        for c0 in range(0, vocab, chunk):
            c1 = min(vocab, c0 + chunk)
            logits = gemm_nt(h, weight[c0:c1], None if bias is None else bias[c0:c1],
                             out_dtype=torch.float32)
            ext.lse_chunk_update(logits, flat_ids, run_max, run_sum, target, c0, float(temperature))
        lse = run_max + torch.log(run_sum)
        ctx.save_for_backward(h, weight, bias if bias is not None else h.new_zeros(0), flat_ids, lse)
        ctx.has_bias = bias is not None
        ctx.temperature, ctx.chunk = float(temperature), int(chunk)
        ctx.hidden_shape = hidden.shape
        return (target - lse).view(ids.shape)

    @staticmethod
    def backward(ctx, g):
        from visionrl_b200.ops import _ext
        from visionrl_b200.ops.linear import gemm_nn, gemm_nt, gemm_tn

        ext = _ext.load()
        h, weight, bias, flat_ids, lse = ctx.saved_tensors
        bias = bias if ctx.has_bias else None
        gflat = g.reshape(-1).contiguous().float()
        vocab = weight.shape[0]
        need_w = ctx.needs_input_grad[1]
        gh = torch.zeros(h.shape, device=h.device, dtype=torch.float32)
        gw = torch.empty_like(weight) if need_w else None
        gb = torch.empty_like(bias) if (bias is not None and ctx.needs_input_grad[2]) else None
        for c0 in range(0, vocab, ctx.chunk):
            c1 = min(vocab, c0 + ctx.chunk)
            logits = gemm_nt(h, weight[c0:c1], None if bias is None else bias[c0:c1],
                             out_dtype=torch.float32)
            dl = ext.softmax_grad_chunk(logits, flat_ids, lse, gflat, c0, ctx.temperature)
            gh += gemm_nn(dl, weight[c0:c1]).float()
            if need_w:
                gw[c0:c1] = gemm_tn(dl, h)
            if gb is not None:
                gb[c0:c1] = ext.colsum(dl).to(gb.dtype)
        return gh.to(h.dtype).view(ctx.hidden_shape), gw, gb, None, None, None


def fused_head_log_probs(hidden, weight, bias, ids, temperature: float = 1.0, chunk: int = 4096):
    from visionrl_b200.ops import _ext

    if (hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and hidden.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and chunk % 8 == 0
            and _ext.kernels_enabled() and _ext.has("lse_chunk_update")):
        if _ext.has("head_logprob_fwd") and hidden.shape[-1] % 8 == 0 and not _CHUNKED_FOLD:
            return _HeadLogProbFn.apply(hidden, weight, bias, ids, temperature, chunk)
        return _FusedHeadLogProbFn.apply(hidden, weight, bias, ids, temperature, chunk)
    return fused_head_log_probs_reference(hidden, weight, bias, ids, temperature)
