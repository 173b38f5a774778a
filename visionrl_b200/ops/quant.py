"""Weight-only int4 linear layers for autoregressive decode (kernel K9 and its oracle).

Weights are quantised symmetrically per ``(output row, group of 128 inputs)``:
``code = clamp(round(w / s) + 8, 0, 15)`` with ``s = max|w| / 7``; eight codes are packed into
one int32 (lowest input index in the low nibble).  Decode batches (at most 32 rows) read the
packed weights once per step, which quarters the bytes a bf16 layer moves.  The reference
implementation has no quantised path (its decode linears are bf16 library GEMMs,
``vrl/models/families/janus_pro/policy.py:673-696``).
"""

from __future__ import annotations

import torch
from torch import nn

GROUP = 128


def quantize_int4(weight: torch.Tensor, group: int = GROUP):
    """``weight[N, K]`` → ``(packed int32 [N, K/8], scales bf16 [N, K/group])``."""
    n, k = weight.shape
    if k % group or k % 8:
        raise ValueError(f"int4 quantisation needs K ({k}) to be a multiple of {group}")
    w = weight.detach().float().view(n, k // group, group)
    scales = (w.abs().amax(dim=-1) / 7.0).clamp_min(1e-8)
    scales = scales.to(torch.bfloat16)
    codes = torch.clamp(torch.round(w / scales.float().unsqueeze(-1)) + 8, 0, 15).to(torch.int64)
    codes = codes.view(n, k // 8, 8)
    shifts = torch.arange(8, device=weight.device, dtype=torch.int64) * 4
    packed = (codes << shifts).sum(dim=-1)
    packed = torch.where(packed >= 2**31, packed - 2**32, packed).to(torch.int32)
    return packed.contiguous(), scales.contiguous()


def dequantize_int4(packed: torch.Tensor, scales: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    n = packed.shape[0]
    words = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=packed.device, dtype=torch.int64) * 4
    codes = ((words.unsqueeze(-1) >> shifts) & 15).view(n, -1).float() - 8.0
    k = codes.shape[1]
    w = codes.view(n, k // group, group) * scales.float().unsqueeze(-1)
    return w.view(n, k)


def int4_linear_reference(x, packed, scales, bias=None, group: int = GROUP):
    w = dequantize_int4(packed, scales, group)
    y = x.float() @ w.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def int4_linear(x, packed, scales, bias=None, group: int = GROUP):
    """``x[..., K]`` times the dequantised ``[N, K]`` weight; kernel paths for decode-sized
    batches on CUDA (≤ 64 rows on the tensor cores, else the CUDA-core GEMV or the oracle)."""
    from visionrl_b200.ops import _ext

    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    on_gpu = x2.is_cuda and x2.dtype == torch.bfloat16 and _ext.kernels_enabled()
    if (on_gpu and 1 <= x2.shape[0] <= 64 and x2.shape[1] % 64 == 0 and group % 64 == 0
            and _ext.has("int4_gemm")):
        # tensor-core path: codes are dequantised inside the SM and fed to tcgen05.mma
        y = _ext.load().int4_gemm(x2.contiguous(), packed, scales, bias, int(group))
    elif (on_gpu and x2.shape[0] <= 32 and x2.shape[1] % 256 == 0 and _ext.has("int4_gemv")):
        y = _ext.load().int4_gemv(x2.contiguous(), packed, scales, bias, int(group))
    else:
        y = int4_linear_reference(x2, packed, scales, bias, group)
    return y.view(*lead, -1)


class Int4Linear(nn.Module):
    """Frozen int4 copy of a linear layer (inference only)."""

    def __init__(self, linear: nn.Module, group: int = GROUP):
        super().__init__()
        weight = linear.weight
        packed, scales = quantize_int4(weight, group)
        self.register_buffer("qweight", packed)
        self.register_buffer("scales", scales)
        bias = getattr(linear, "bias", None)
        self.register_buffer("bias", bias.detach().clone() if bias is not None else None)
        self.group = group
        self.in_features, self.out_features = weight.shape[1], weight.shape[0]

    def forward(self, x):
        return int4_linear(x, self.qweight, self.scales, self.bias, self.group)


def build_int4_shadow(module: nn.Module, group: int = GROUP) -> dict[str, Int4Linear]:
    """Int4 copies of every plain linear under ``module`` whose input width allows it.

    Returns ``{qualified name: Int4Linear}``; the caller decides when to route through them
    (decode steps) and must rebuild the shadow after the weights change.
    """
    out: dict[str, Int4Linear] = {}
    for name, sub in module.named_modules():
        weight = getattr(sub, "weight", None)
        if (isinstance(sub, nn.Linear) or type(sub).__name__ in ("Linear", "LoRALinear")) \
                and weight is not None and weight.dim() == 2 and weight.shape[1] % 256 == 0:
            out[name] = Int4Linear(sub, group)
    return out


__all__ = ["GROUP", "Int4Linear", "build_int4_shadow", "dequantize_int4", "int4_linear",
           "int4_linear_reference", "quantize_int4"]
