"""Token log-probabilities (kernel K7 and its oracle).

``token_log_probs(logits, ids, T)`` = ``log_softmax(logits / T)[ids]`` in fp32.
``fused_head_log_probs(hidden, weight, bias, ids, T)`` computes the same quantity
from the pre-head hidden states, tiling the head GEMM over the vocabulary with an
online log-sum-exp so the ``[rows, vocab]`` fp32 logits never exist in HBM.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


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


def fused_head_log_probs(hidden, weight, bias, ids, temperature: float = 1.0):
    return fused_head_log_probs_reference(hidden, weight, bias, ids, temperature)
