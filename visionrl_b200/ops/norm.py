"""Normalisation kernels (K3) and their oracles.

* :func:`adaln_layernorm` — affine-free LayerNorm followed by the adaLN
  modulation ``y = LN(x) * (1 + scale[b]) + shift[b]`` for ``x[B, S, D]``.
* :func:`rmsnorm` — ``y = x / sqrt(mean(x^2) + eps) * weight`` over the last dim.
* :func:`layernorm` — affine LayerNorm over the last dim.

CUDA bf16 inputs run one-row-per-warp sm_100a kernels (single pass over the
row in registers, fp32 statistics); CPU tensors use the PyTorch formulas.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def adaln_layernorm_reference(x, shift, scale, eps: float = 1e-6):
    y = F.layer_norm(x.float(), (x.shape[-1],), None, None, eps)
    y = y * (1 + scale.float().unsqueeze(1)) + shift.float().unsqueeze(1)
    return y.to(x.dtype)


def rmsnorm_reference(x, weight, eps: float = 1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


class _AdaLNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, scale, eps):
        from visionrl_b200.ops import _ext

        y, mean, rstd = _ext.load().adaln_fwd(x.contiguous(), shift, scale, float(eps))
        ctx.save_for_backward(x, scale, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        x, scale, mean, rstd = ctx.saved_tensors
        gx, gshift, gscale = _ext.load().adaln_bwd(gy.contiguous(), x.contiguous(), scale, mean,
                                                   rstd)
        return gx, gshift.to(scale.dtype), gscale.to(scale.dtype), None


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        from visionrl_b200.ops import _ext

        y, rstd = _ext.load().rmsnorm_fwd(x.contiguous(), weight.contiguous(), float(eps))
        ctx.save_for_backward(x, weight, rstd)
        return y

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        x, weight, rstd = ctx.saved_tensors
        gx, gw = _ext.load().rmsnorm_bwd(gy.contiguous(), x.contiguous(), weight.contiguous(), rstd)
        return gx, gw.to(weight.dtype), None


def _kernel_ok(x) -> bool:
    from visionrl_b200.ops import _ext

    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
            and x.shape[-1] <= 8192 and _ext.kernels_enabled())


def adaln_layernorm(x, shift, scale, eps: float = 1e-6):
    if _kernel_ok(x) and x.dim() == 3:
        return _AdaLNFn.apply(x, shift, scale, eps)
    return adaln_layernorm_reference(x, shift, scale, eps)


def rmsnorm(x, weight, eps: float = 1e-6):
    if _kernel_ok(x) and weight is not None:
        return _RMSNormFn.apply(x, weight, eps)
    return rmsnorm_reference(x, weight, eps)


def layernorm(x, weight, bias, eps: float = 1e-5):
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def group_norm_silu(x, norm, apply_silu: bool = True):
    """``silu(group_norm(x))`` for a ``torch.nn.GroupNorm`` module ``norm``.

    Channels-last bf16 CUDA activations outside autograd (the frozen decoders of the reward
    path) take one statistics pass and one fused normalise(+SiLU) pass of the sm_100a kernel;
    everything else evaluates the module and the activation separately.
    """
    import torch.nn.functional as F

    from visionrl_b200.ops import _ext

    c = x.shape[1] if x.dim() == 4 else 0
    if (x.dim() == 4 and x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled()
            and norm.affine and c % 8 == 0 and 256 % (c // 8) == 0 and c // 8 <= 256
            and x.is_contiguous(memory_format=torch.channels_last)
            and _ext.kernels_enabled() and _ext.has("groupnorm_nhwc")):
        return _ext.load().groupnorm_nhwc(x, norm.weight, norm.bias, int(norm.num_groups),
                                          float(norm.eps), bool(apply_silu))
    y = norm(x)
    return F.silu(y) if apply_silu else y
