"""MMDiT: joint image/text transformer with adaLN-Zero modulation (SD3.5 shape).

Two token streams (image patches, text context) keep separate weights and meet
in one joint attention per block.  ``q``/``k`` are RMS-normalised per head.  The
last block's text stream only feeds attention ("context pre-only").  The same
class with small dimensions is the tiny DiT of the CPU end-to-end configuration.
Per block and stream: adaLN-LayerNorm → fused QKV GEMM → head split + QK norm →
joint attention → out-projection with gate·residual epilogue → adaLN-LayerNorm →
MLP (GELU-tanh epilogue, then gate·residual epilogue).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from visionrl_b200.models.nn.layers import (
    AdapterMixin,
    Linear, LoRALinear, MLP, TimestepEmbedder, merge_heads, sdpa,
)
from visionrl_b200.ops import norm as norm_ops
from visionrl_b200.ops.qkv import joint_qkv_prepare, qkv_prepare


@dataclass
class MMDiTConfig:
    num_layers: int = 24
    hidden_size: int = 1536
    num_heads: int = 24
    patch_size: int = 2
    in_channels: int = 16
    context_dim: int = 4096
    pooled_dim: int = 2048
    mlp_ratio: float = 4.0
    max_grid: int = 192          # largest latent side (in patches) of the position table
    qk_norm: bool = True
    moe_experts: int = 0         # > 0: the image-stream FFN is a routed mixture of this many experts
    moe_top_k: int = 2

    @classmethod
    def from_dict(cls, d: dict) -> "MMDiTConfig":
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: d[k] for k in keys if k in d})


def sincos_2d(dim: int, grid: int) -> torch.Tensor:
    """Fixed 2-D sine/cosine table ``[grid*grid, dim]`` (half of ``dim`` per axis)."""
    quarter = dim // 4
    omega = 1.0 / (10000 ** (torch.arange(quarter, dtype=torch.float64) / quarter))
    pos = torch.arange(grid, dtype=torch.float64)
    ang = pos[:, None] * omega[None]
    axis = torch.cat([torch.sin(ang), torch.cos(ang)], dim=1)
    row = axis[:, None, :].expand(grid, grid, -1)
    col = axis[None, :, :].expand(grid, grid, -1)
    return torch.cat([row, col], dim=-1).reshape(grid * grid, -1).float()


class StreamAttention(nn.Module):
    """QKV / output projections of one stream.  ``qkv`` is one fused GEMM; the LoRA
    target names ``to_q``/``to_k``/``to_v``/``to_out.0`` (image) and
    ``add_*_proj``/``to_add_out`` (text) address the same sub-matrices."""

    def __init__(self, dim: int, heads: int, qk_norm: bool, has_out: bool = True):
        super().__init__()
        self.heads = heads
        self.qkv = LoRALinear(dim, 3 * dim)
        self.q_norm = nn.Parameter(torch.ones(dim // heads)) if qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(dim // heads)) if qk_norm else None
        self.out = LoRALinear(dim, dim) if has_out else None

    def set_aliases(self, qkv_names: tuple, out_name: str) -> None:
        self.qkv.lora_aliases = qkv_names
        if self.out is not None:
            self.out.lora_aliases = (out_name,)

    def project(self, x):
        return qkv_prepare(self.qkv(x), self.heads, self.q_norm, self.k_norm)


class _MoEAdapter(nn.Module):
    """Routed feed-forward block with the calling convention of :class:`MLP`."""

    def __init__(self, dim: int, hidden: int, experts: int, top_k: int):
        super().__init__()
        from visionrl_b200.ops.moe import MoEFFN

        self.ffn = MoEFFN(dim, hidden, experts, min(top_k, experts))

    def forward(self, x, gate=None, residual=None):
        from visionrl_b200.ops.linear import linear_epilogue

        return linear_epilogue(self.ffn(x), None, gate, residual)


class _SplitStreams(torch.autograd.Function):
    """Joint ``[B, Sx + Sc, D]`` activations → contiguous image and text parts.

    The gradient is one concatenation instead of two zero-filled full-size tensors and an add.
    """

    @staticmethod
    def forward(ctx, o, sx):
        ctx.sx = sx
        return o[:, :sx].contiguous(), o[:, sx:].contiguous()

    @staticmethod
    def backward(ctx, gx, gc):
        return torch.cat([gx, gc], dim=1), None


class JointBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, context_pre_only: bool = False):
        super().__init__()
        d, hidden = cfg.hidden_size, int(cfg.hidden_size * cfg.mlp_ratio)
        self.context_pre_only = context_pre_only
        self.mod_x = Linear(d, 6 * d, init_std=0.02)
        self.mod_c = Linear(d, (2 if context_pre_only else 6) * d, init_std=0.02)
        self.attn_x = StreamAttention(d, cfg.num_heads, cfg.qk_norm)
        self.attn_c = StreamAttention(d, cfg.num_heads, cfg.qk_norm, has_out=not context_pre_only)
        self.attn_x.set_aliases(("to_q", "to_k", "to_v"), "to_out.0")
        self.attn_c.set_aliases(("add_q_proj", "add_k_proj", "add_v_proj"), "to_add_out")
        self.mlp_x = _MoEAdapter(d, hidden, cfg.moe_experts, cfg.moe_top_k) if cfg.moe_experts > 0 \
            else MLP(d, hidden)
        self.mlp_c = None if context_pre_only else MLP(d, hidden)

    def forward(self, x, c, temb_act):
        sx = x.shape[1]
        mx = self.mod_x(temb_act).chunk(6, dim=-1)
        mc = self.mod_c(temb_act).chunk(2 if self.context_pre_only else 6, dim=-1)
        ax, ac = self.attn_x, self.attn_c
        q, k, v = joint_qkv_prepare(
            ax.qkv(norm_ops.adaln_layernorm(x, mx[0], mx[1])),
            ac.qkv(norm_ops.adaln_layernorm(c, mc[0], mc[1])),
            ax.heads, (ax.q_norm, ax.k_norm), (ac.q_norm, ac.k_norm))
        ox, oc = _SplitStreams.apply(merge_heads(sdpa(q, k, v)), sx)
        x = self.attn_x.out(ox, gate=mx[2], residual=x)
        x = self.mlp_x(norm_ops.adaln_layernorm(x, mx[3], mx[4]), gate=mx[5], residual=x)
        if self.context_pre_only:
            return x, None
        c = self.attn_c.out(oc, gate=mc[2], residual=c)
        c = self.mlp_c(norm_ops.adaln_layernorm(c, mc[3], mc[4]), gate=mc[5], residual=c)
        return x, c


class MMDiT(AdapterMixin, nn.Module):
    def __init__(self, cfg: MMDiTConfig):
        super().__init__()
        self.cfg = cfg
        d, p = cfg.hidden_size, cfg.patch_size
        self.patch_embed = Linear(cfg.in_channels * p * p, d)
        self.register_buffer("pos_table", sincos_2d(d, cfg.max_grid), persistent=False)
        self.time_embed = TimestepEmbedder(d)
        self.pooled_embed = MLP(cfg.pooled_dim, d, act="silu")
        self.pooled_embed.fc2 = Linear(d, d)
        self.context_embed = Linear(cfg.context_dim, d)
        self.blocks = nn.ModuleList(
            JointBlock(cfg, context_pre_only=(i == cfg.num_layers - 1))
            for i in range(cfg.num_layers)
        )
        self.final_mod = Linear(d, 2 * d, init_std=0.02)
        self.final_proj = Linear(d, cfg.in_channels * p * p, init_std=0.02)
        self.gradient_checkpointing = False

    # -- helpers -----------------------------------------------------------------
    def enable_gradient_checkpointing(self, flag: bool = True) -> None:
        self.gradient_checkpointing = flag

    def patchify(self, latents):
        b, ch, h, w = latents.shape
        p = self.cfg.patch_size
        x = latents.view(b, ch, h // p, p, w // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(b, (h // p) * (w // p), ch * p * p), h // p, w // p

    def unpatchify(self, x, gh, gw):
        b = x.shape[0]
        p, ch = self.cfg.patch_size, self.cfg.in_channels
        x = x.view(b, gh, gw, ch, p, p).permute(0, 3, 1, 4, 2, 5)
        return x.reshape(b, ch, gh * p, gw * p)

    def pos_embed(self, gh, gw, dtype):
        g = self.cfg.max_grid
        top, left = (g - gh) // 2, (g - gw) // 2
        table = self.pos_table.view(g, g, -1)[top:top + gh, left:left + gw]
        return table.reshape(1, gh * gw, -1).to(dtype)

    # -- forward -----------------------------------------------------------------
    def forward(self, latents, timestep, context, pooled):
        """``latents[B,C,H,W]``, ``timestep[B]``, ``context[B,L,Dc]``, ``pooled[B,Dp]`` → velocity."""
        dtype = self.patch_embed.weight.dtype
        tokens, gh, gw = self.patchify(latents.to(dtype))
        x = self.patch_embed(tokens) + self.pos_embed(gh, gw, dtype)
        temb = self.time_embed(timestep, dtype) + self.pooled_embed(pooled.to(dtype))
        temb_act = torch.nn.functional.silu(temb)
        c = self.context_embed(context.to(dtype))
        for block in self.blocks:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                x, c = checkpoint(block, x, c, temb_act, use_reentrant=False)
            else:
                x, c = block(x, c, temb_act)
        scale, shift = self.final_mod(temb_act).chunk(2, dim=-1)
        x = self.final_proj(norm_ops.adaln_layernorm(x, shift, scale))
        return self.unpatchify(x, gh, gw)

    def flops_per_sample(self, grid_tokens: int, context_tokens: int) -> float:
        """Forward multiply-add FLOPs (×2) of one sample, for roofline reports."""
        cfg = self.cfg
        d, hid = cfg.hidden_size, int(cfg.hidden_size * cfg.mlp_ratio)
        per_tok = 2 * (3 * d * d + d * d + 2 * d * hid)
        s = grid_tokens + context_tokens
        attn = 4 * s * s * d
        return cfg.num_layers * (per_tok * s + attn)
