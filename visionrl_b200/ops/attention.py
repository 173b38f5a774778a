"""Attention entry points (kernels K2 and K8) with a PyTorch oracle.

``attention(q, k, v)`` takes ``[B, H, S, D]`` tensors and returns ``[B, H, S, D]``.
The oracle is ``softmax(q k^T / sqrt(D)) v`` in fp32.
"""

from __future__ import annotations

import math
import os

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


def _has_backward() -> bool:
    from visionrl_b200.ops import _ext

    return _ext.has("flash_attn_bwd")


def flash_attention_forward(q, k, v, scale: float, causal: bool = False, variant: int = 0):
    """tcgen05 forward kernel: returns ``(out, lse)`` with ``lse[B, H, S]`` in natural log.

    ``causal``: query row ``r`` attends keys ``0 … r + (Skv - Sq)``.  ``variant`` selects the kernel
    (0 = default for the shape, 1 = register-accumulating, 2 = lazy-rescale) for benchmarks."""
    from visionrl_b200.ops import _ext

    out, lse = _ext.load().flash_attn_fwd(q, k, v, float(scale), bool(causal), int(variant))
    return out, lse


def flash_attention_backward(dout, q, k, v, out, lse, scale: float, causal: bool = False):
    """tcgen05 backward kernels (delta pre-pass, dK/dV pass, dQ pass): returns ``(dq, dk, dv)``."""
    from visionrl_b200.ops import _ext

    return _ext.load().flash_attn_bwd(dout, q, k, v, out, lse, float(scale), bool(causal))


class _FlashAttnFn(torch.autograd.Function):
    """Differentiable attention on the sm_100a kernels: forward saves ``out`` and the row
    log-sum-exp, backward recomputes the probabilities tile by tile."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal=False):
        out, lse = flash_attention_forward(q, k, v, scale, causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale, ctx.causal = scale, bool(causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_attention_backward(dout, q, k, v, out, lse, ctx.scale, ctx.causal)
        return dq, dk, dv, None, None


# Which implementation differentiable calls use: "own" = the tcgen05 forward/backward pair above,
# "library" = torch's fused scaled_dot_product_attention.  Chosen per process.
_BACKWARD_IMPL = os.environ.get("VRL_ATTENTION_BACKWARD", "own")


def set_backward_impl(name: str) -> None:
    global _BACKWARD_IMPL
    if name not in ("own", "library"):
        raise ValueError(f"attention backward implementation must be 'own' or 'library', got {name!r}")
    _BACKWARD_IMPL = name


def backward_impl() -> str:
    return _BACKWARD_IMPL


def attention(q, k, v, causal: bool = False, scale: float | None = None):
    """Bidirectional (or causal) attention over ``[B, H, S, D]``.

    bf16 calls with head dimension 64 or 128 — bidirectional or causal (``Sq <= Skv``, the last
    query aligned with the last key) — run the hand-written sm_100a kernels: the forward alone when
    no gradient is needed (rollout sampling, prefill, frozen-reference passes, reward towers), the
    forward/backward pair otherwise.  Other shapes use the library's fused attention.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if _native_ok(q, k, v) and (not causal or q.shape[2] <= k.shape[2]):
        if not needs_grad:
            return flash_attention_forward(q, k, v, scale, causal)[0]
        if _BACKWARD_IMPL == "own" and _has_backward():
            return _FlashAttnFn.apply(q, k, v, scale, causal)
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
