"""Element-wise part of the flow-matching SDE step (kernel K5 and its oracle).

Inputs are fp32.  ``a``, ``b``, ``scale`` and ``dt`` are per-sample scalars such
that ``mu = a*x + b*v`` and ``x' = mu + scale*eps``.  ``gaussian=True`` selects the
normalised Gaussian log-density (``sde``), ``False`` the ``-(x'-mu)^2`` score of
the ``cps`` sampler.  The log-probability is the mean over all non-batch
elements.  CUDA tensors go through the fused sm_100a kernel (one read of ``v``,
``x`` and the noise / recorded sample, one write of ``x'`` and ``mu``, block
reduction of the log-density); CPU tensors use :func:`sde_step_reference`.
"""

from __future__ import annotations

import math

import torch

_LOG_SQRT_2PI = math.log(math.sqrt(2 * math.pi))


def sde_step_reference(v, x, a, b, scale, dt, prev_sample=None, noise=None,
                       deterministic=False, gaussian=True):
    view = (-1,) + (1,) * (x.ndim - 1)
    a, b, scale, dt = (t.view(view) for t in (a, b, scale, dt))
    mean = a * x + b * v
    if prev_sample is None:
        prev_sample = mean + scale * noise
    if deterministic:
        prev_sample = x + dt * v
    diff2 = (prev_sample.detach() - mean) ** 2
    if gaussian:
        log_prob = -diff2 / (2 * scale**2) - torch.log(scale) - _LOG_SQRT_2PI
    else:
        log_prob = -diff2
    return prev_sample, log_prob.mean(dim=tuple(range(1, x.ndim))), mean


class _FusedSDEStep(torch.autograd.Function):
    """CUDA path.  Gradients reach ``v`` (and ``x``) through ``mu`` only."""

    @staticmethod
    def forward(ctx, v, x, a, b, scale, dt, prev_sample, noise, deterministic, gaussian):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        out_prev, log_prob, mean = ext.sde_step_fwd(
            v.contiguous(), x.contiguous(), a.contiguous(), b.contiguous(),
            scale.contiguous(), dt.contiguous(),
            None if prev_sample is None else prev_sample.contiguous(),
            None if noise is None else noise.contiguous(),
            bool(deterministic), bool(gaussian),
        )
        ctx.save_for_backward(out_prev, mean, a, b, scale)
        ctx.gaussian = gaussian
        ctx.mark_non_differentiable(out_prev)
        return out_prev, log_prob, mean

    @staticmethod
    def backward(ctx, _g_prev, g_logp, g_mean):
        from visionrl_b200.ops import _ext

        out_prev, mean, a, b, scale = ctx.saved_tensors
        ext = _ext.load()
        g_logp = torch.zeros(mean.shape[0], device=mean.device) if g_logp is None else g_logp
        g_v, g_x = ext.sde_step_bwd(
            out_prev, mean, a, b, scale, g_logp.contiguous().float(),
            None if g_mean is None else g_mean.contiguous(), bool(ctx.gaussian),
        )
        return g_v, g_x, None, None, None, None, None, None, None, None


def sde_step(v, x, a, b, scale, dt, prev_sample=None, noise=None,
             deterministic=False, gaussian=True):
    """Returns ``(prev_sample, log_prob[B], prev_sample_mean)``."""
    from visionrl_b200.ops import _ext

    if v.is_cuda and _ext.kernels_enabled():
        return _FusedSDEStep.apply(v, x, a, b, scale, dt, prev_sample, noise,
                                   deterministic, gaussian)
    return sde_step_reference(v, x, a, b, scale, dt, prev_sample, noise, deterministic, gaussian)
