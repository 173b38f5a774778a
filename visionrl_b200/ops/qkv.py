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


def _heads_first(t):
    """Token-major ``[B, S, H, Dh]`` buffer viewed as ``[B, H, S, Dh]``."""
    return t.transpose(1, 2)


class _QKVPrepFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, cos, sin, heads, eps):
        from visionrl_b200.ops import _ext

        q, k, v, rstd = _ext.load().qkv_prepare_fwd(qkv.contiguous(), q_weight, k_weight, cos, sin,
                                                    int(heads), float(eps), None, None, None, 0)
        ctx.save_for_backward(qkv, q_weight, k_weight, cos, sin, rstd)
        ctx.heads = heads
        return _heads_first(q), _heads_first(k), _heads_first(v)

    @staticmethod
    def backward(ctx, gq, gk, gv):
        from visionrl_b200.ops import _ext

        qkv, q_weight, k_weight, cos, sin, rstd = ctx.saved_tensors
        gqkv, gqw, gkw = _ext.load().qkv_prepare_bwd(
            gq, gk, gv, qkv, q_weight, k_weight, cos, sin, rstd, int(ctx.heads), 0)
        gqw = None if q_weight is None else gqw.to(q_weight.dtype)
        gkw = None if k_weight is None else gkw.to(k_weight.dtype)
        return gqkv, gqw, gkw, None, None, None, None


class _JointQKVPrepFn(torch.autograd.Function):
    """Two token streams written into ONE joint ``[B, Sa + Sb, H, Dh]`` q/k/v buffer.

    The joint-attention block of an MMDiT attends over the concatenation of image and text
    tokens; writing both streams straight into the joint buffer removes the three
    concatenation copies of the forward pass and the matching slice copies of the backward.
    """

    @staticmethod
    def forward(ctx, qkv_a, qkv_b, qw_a, kw_a, qw_b, kw_b, heads, eps):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        b, sa, d3 = qkv_a.shape
        sb = qkv_b.shape[1]
        dh = d3 // (3 * heads)
        q = torch.empty(b, sa + sb, heads, dh, device=qkv_a.device, dtype=qkv_a.dtype)
        k, v = torch.empty_like(q), torch.empty_like(q)
        *_, rstd_a = ext.qkv_prepare_fwd(qkv_a.contiguous(), qw_a, kw_a, None, None, int(heads),
                                         float(eps), q, k, v, 0)
        *_, rstd_b = ext.qkv_prepare_fwd(qkv_b.contiguous(), qw_b, kw_b, None, None, int(heads),
                                         float(eps), q, k, v, sa)
        ctx.save_for_backward(qkv_a, qkv_b, qw_a, kw_a, qw_b, kw_b, rstd_a, rstd_b)
        ctx.heads, ctx.sa = heads, sa
        return _heads_first(q), _heads_first(k), _heads_first(v)

    @staticmethod
    def backward(ctx, gq, gk, gv):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        qkv_a, qkv_b, qw_a, kw_a, qw_b, kw_b, rstd_a, rstd_b = ctx.saved_tensors
        ga, gqw_a, gkw_a = ext.qkv_prepare_bwd(gq, gk, gv, qkv_a, qw_a, kw_a, None, None, rstd_a,
                                               int(ctx.heads), 0)
        gb, gqw_b, gkw_b = ext.qkv_prepare_bwd(gq, gk, gv, qkv_b, qw_b, kw_b, None, None, rstd_b,
                                               int(ctx.heads), int(ctx.sa))

        def cast(g, w):
            return None if w is None else g.to(w.dtype)

        return (ga, gb, cast(gqw_a, qw_a), cast(gkw_a, kw_a), cast(gqw_b, qw_b), cast(gkw_b, kw_b),
                None, None)


def _kernel_ok(qkv, heads: int) -> bool:
    from visionrl_b200.ops import _ext

    dh = qkv.shape[-1] // (3 * heads)
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and dh in (64, 128)
            and qkv.shape[-1] <= 16384 and _ext.kernels_enabled())


def qkv_prepare(qkv, heads: int, q_weight=None, k_weight=None, eps: float = 1e-6, rope=None):
    if _kernel_ok(qkv, heads):
        cos, sin = rope if rope is not None else (None, None)
        return _QKVPrepFn.apply(qkv, q_weight, k_weight, cos, sin, heads, eps)
    return qkv_prepare_reference(qkv, heads, q_weight, k_weight, eps, rope)


def joint_qkv_prepare(qkv_a, qkv_b, heads: int, norms_a=(None, None), norms_b=(None, None),
                      eps: float = 1e-6):
    """``(q, k, v)`` over the concatenated sequence ``[a | b]`` as ``[B, H, Sa + Sb, Dh]``."""
    if _kernel_ok(qkv_a, heads) and _kernel_ok(qkv_b, heads):
        return _JointQKVPrepFn.apply(qkv_a, qkv_b, norms_a[0], norms_a[1], norms_b[0], norms_b[1],
                                     heads, eps)
    qa, ka, va = qkv_prepare_reference(qkv_a, heads, norms_a[0], norms_a[1], eps)
    qb, kb, vb = qkv_prepare_reference(qkv_b, heads, norms_b[0], norms_b[1], eps)
    return torch.cat([qa, qb], 2), torch.cat([ka, kb], 2), torch.cat([va, vb], 2)
