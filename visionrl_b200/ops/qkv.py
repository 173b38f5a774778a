"""QKV post-processing (part of kernels K3/K4): head split, per-head RMS norm of
``q`` and ``k``, optional rotary embedding, output in ``[B, H, S, Dh]``.

``qkv`` is the fused projection output ``[B, S, 3*H*Dh]`` ordered (q | k | v).
The norm weights have ``Dh`` elements (per-head norm) or ``H*Dh`` elements (norm over
the whole projection width).  ``rope`` is a ``(cos, sin)`` pair of ``[S, Dh/2]`` fp32 tables applied to
interleaved pairs ``(x[2i], x[2i+1])``.
"""

from __future__ import annotations

import torch

from visionrl_b200.ops.norm import rmsnorm_reference


def apply_rope_reference(x, cos, sin):
    """``x[..., S, Dh]`` rotated pairwise by tables ``[S, Dh/2]``."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    x0, x1 = xf[..., 0], xf[..., 1]
    out = torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)
    return out.reshape(x.shape).to(x.dtype)


def qkv_prepare_reference(qkv, heads: int, q_weight=None, k_weight=None, eps: float = 1e-6,
                          rope=None):
    b, s, d3 = qkv.shape
    dh = d3 // (3 * heads)
    q, k, v = qkv.view(b, s, 3, heads, dh).unbind(2)
    if q_weight is not None and q_weight.numel() == heads * dh and heads > 1:
        # norm over the whole projection width ("across heads", Wan-style)
        q = rmsnorm_reference(q.reshape(b, s, -1), q_weight, eps).view(b, s, heads, dh)
        k = rmsnorm_reference(k.reshape(b, s, -1), k_weight, eps).view(b, s, heads, dh)
    elif q_weight is not None:
        q = rmsnorm_reference(q, q_weight, eps)
        k = rmsnorm_reference(k, k_weight, eps)
    q, k, v = (t.transpose(1, 2) for t in (q, k, v))
    if rope is not None:
        cos, sin = rope
        q = apply_rope_reference(q, cos, sin)
        k = apply_rope_reference(k, cos, sin)
    return q, k, v


class _QKVPrepFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, cos, sin, heads, eps):
        from visionrl_b200.ops import _ext

        q, k, v, rstd = _ext.load().qkv_prepare_fwd(qkv.contiguous(), q_weight, k_weight, cos, sin,
                                                    int(heads), float(eps))
        ctx.save_for_backward(qkv, q_weight, k_weight, cos, sin, rstd)
        ctx.heads = heads
        return q, k, v

    @staticmethod
    def backward(ctx, gq, gk, gv):
        from visionrl_b200.ops import _ext

        qkv, q_weight, k_weight, cos, sin, rstd = ctx.saved_tensors
        gqkv, gqw, gkw = _ext.load().qkv_prepare_bwd(
            gq.contiguous(), gk.contiguous(), gv.contiguous(), qkv, q_weight, k_weight, cos, sin,
            rstd, int(ctx.heads))
        gqw = None if q_weight is None else gqw.to(q_weight.dtype)
        gkw = None if k_weight is None else gkw.to(k_weight.dtype)
        return gqkv, gqw, gkw, None, None, None, None


def qkv_prepare(qkv, heads: int, q_weight=None, k_weight=None, eps: float = 1e-6, rope=None):
    dh = qkv.shape[-1] // (3 * heads)
    from visionrl_b200.ops import _ext

    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and dh in (64, 128)
            and qkv.shape[-1] <= 16384 and _ext.kernels_enabled()):
        cos, sin = rope if rope is not None else (None, None)
        return _QKVPrepFn.apply(qkv, q_weight, k_weight, cos, sin, heads, eps)
    return qkv_prepare_reference(qkv, heads, q_weight, k_weight, eps, rope)
