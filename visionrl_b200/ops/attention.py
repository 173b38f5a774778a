"""Attention entry points (kernels K2 and K8) with a PyTorch oracle.

``attention(q, k, v)`` takes ``[B, H, S, D]`` tensors and returns ``[B, H, S, D]``.
The oracle is ``softmax(q k^T / sqrt(D)) v`` in fp32.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def attention_reference(q, k, v, causal: bool = False, scale: float | None = None):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v.float()).to(q.dtype)


def _native_ok(q, k, v) -> bool:
    from visionrl_b200.ops import _ext

    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and q.dim() == 4 and q.shape[-1] in (64, 128) and k.shape[-1] == q.shape[-1]
            and v.shape == k.shape and q.shape[0] * q.shape[1] <= 65535
            and _ext.kernels_enabled() and _ext.has("flash_attn_fwd"))


def flash_attention_forward(q, k, v, scale: float):
    """tcgen05 forward kernel: returns ``(out, lse)`` with ``lse[B, H, S]`` in natural log."""
    from visionrl_b200.ops import _ext

    out, lse = _ext.load().flash_attn_fwd(q, k, v, float(scale))
    return out, lse


def attention(q, k, v, causal: bool = False, scale: float | None = None):
    """Bidirectional (or causal) attention over ``[B, H, S, D]``.

    Calls that need no gradient (rollout sampling, frozen-reference passes, reward towers) run
    the hand-written sm_100a forward kernel; differentiable calls use the library's fused
    forward/backward pair until the tcgen05 backward lands.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if not causal and not needs_grad and _native_ok(q, k, v):
        return flash_attention_forward(q, k, v, scale)[0]
    if q.is_cuda:
        return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)
    return attention_reference(q, k, v, causal, scale)


def decode_attention_reference(q, k_cache, v_cache, valid, length: int, scale: float | None = None):
    """One query position per row against a static cache.

    ``q[R, H, 1, D]``, ``k_cache``/``v_cache`` ``[R, H, max_len, D]``, ``valid[R, max_len]`` marks
    usable key positions, ``length`` is the number of filled positions.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    k = k_cache[:, :, :length].float()
    v = v_cache[:, :, :length].float()
    s = torch.matmul(q.float(), k.transpose(-1, -2)) * scale
    s = s.masked_fill(~valid[:, None, None, :length], float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v).to(q.dtype)


def decode_attention(q, k_cache, v_cache, valid, length: int, scale: float | None = None):
    from visionrl_b200.ops import _ext

    if (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and _ext.kernels_enabled()
            and _ext.has("decode_attention")):
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        return _ext.load().decode_attention(q.contiguous(), k_cache, v_cache, valid, int(length),
                                            float(scale))
    return decode_attention_reference(q, k_cache, v_cache, valid, length, scale)
