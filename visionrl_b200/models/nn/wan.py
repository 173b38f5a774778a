"""Wan-2.1-shape video DiT: self-attention with 3-D RoPE, cross-attention to text
tokens and a GELU FFN, modulated by a learned table plus the time embedding.

Tokens are ``(t, h, w)`` patches in row-major order.  Rotary frequencies split
the head dimension into a temporal part and two spatial parts
(``Dh - 2*(Dh//3)``, ``Dh//3``, ``Dh//3`` channels).  ``seq_shard=(rank, size)``
restricts a forward to one contiguous slice of the token sequence; attention
then goes through the Ulysses head/sequence exchange of
:mod:`visionrl_b200.parallel.ulysses`.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from visionrl_b200.models.nn.layers import (
    AdapterMixin,
    LayerNorm, Linear, LoRALinear, MLP, TimestepEmbedder, merge_heads, sdpa, split_heads,
)
from visionrl_b200.ops import norm as norm_ops
from visionrl_b200.ops.qkv import apply_rope_reference, qkv_prepare


@dataclass
class WanConfig:
    num_layers: int = 30
    hidden_size: int = 1536
    num_heads: int = 12
    ffn_dim: int = 8960
    patch_size: tuple = (1, 2, 2)
    in_channels: int = 16
    out_channels: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    extra_in_channels: int = 0      # conditioning channels concatenated to the latent
    rope_theta: float = 10000.0

    @classmethod
    def from_dict(cls, d: dict) -> "WanConfig":
        keys = cls.__dataclass_fields__.keys()
        out = {k: d[k] for k in keys if k in d}
        if "patch_size" in out:
            out["patch_size"] = tuple(out["patch_size"])
        if "in_channels" in out and "out_channels" not in out:
            out["out_channels"] = out["in_channels"]
        return cls(**out)


def rope_3d_tables(grid: tuple, head_dim: int, theta: float, device) -> tuple:
    """``(cos, sin)`` of shape ``[T*H*W, head_dim/2]`` for a ``(T, H, W)`` token grid."""
    t, h, w = grid
    d_h = d_w = 2 * (head_dim // 6)
    d_t = head_dim - d_h - d_w
    angles = []
    for n, d, reps in ((t, d_t, (1, h, w)), (h, d_h, (t, 1, w)), (w, d_w, (t, h, 1))):
        freqs = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=device) / d))
        a = torch.arange(n, dtype=torch.float64, device=device)[:, None] * freqs[None]
        shape = [1, 1, 1, d // 2]
        axis = {0: 0, 1: 1, 2: 2}[len(angles)]
        shape[axis] = n
        angles.append(a.view(*shape).expand(t, h, w, d // 2))
    ang = torch.cat(angles, dim=-1).reshape(t * h * w, head_dim // 2)
    return torch.cos(ang).float(), torch.sin(ang).float()


class WanSelfAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.qkv = LoRALinear(dim, 3 * dim)
        self.q_norm = nn.Parameter(torch.ones(dim))
        self.k_norm = nn.Parameter(torch.ones(dim))
        self.out = LoRALinear(dim, dim)
        self.qkv.lora_aliases = ("to_q", "to_k", "to_v")
        self.out.lora_aliases = ("to_out.0",)

    def forward(self, x, rope, gate, residual, sp=None):
        qkv = self.qkv(x)
        if sp is not None and sp.can_fuse(qkv, self.heads):
            # head split + QK norm + RoPE store straight into the head owners' buffers, attention
            # stores straight into the token owners' buffer: the output projection reads a view
            o = sp.fused_attention(qkv, self.heads, self.q_norm, self.k_norm, rope)
            return self.out(o, gate=gate, residual=residual)
        q, k, v = qkv_prepare(qkv, self.heads, self.q_norm, self.k_norm, rope=rope)
        if sp is not None:
            o = sp.attention(q, k, v)
        else:
            o = sdpa(q, k, v)
        return self.out(merge_heads(o), gate=gate, residual=residual)


class WanCrossAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.q = LoRALinear(dim, dim)
        self.kv = LoRALinear(dim, 2 * dim)
        self.q_norm = nn.Parameter(torch.ones(dim))
        self.k_norm = nn.Parameter(torch.ones(dim))
        self.out = LoRALinear(dim, dim)
        self.q.lora_aliases = ("to_q",)
        self.kv.lora_aliases = ("to_k", "to_v")
        self.out.lora_aliases = ("to_out.0",)

    def forward(self, x, ctx, residual):
        q = norm_ops.rmsnorm(self.q(x), self.q_norm)
        k, v = self.kv(ctx).chunk(2, dim=-1)
        k = norm_ops.rmsnorm(k.contiguous(), self.k_norm)
        o = sdpa(split_heads(q, self.heads), split_heads(k, self.heads),
                 split_heads(v.contiguous(), self.heads))
        return residual + self.out(merge_heads(o))


class WanBlock(nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        d = cfg.hidden_size
        self.mod_table = nn.Parameter(torch.randn(6, d) / d**0.5)
        self.self_attn = WanSelfAttention(d, cfg.num_heads)
        self.cross_norm = LayerNorm(d, eps=1e-6, affine=True)
        self.cross_attn = WanCrossAttention(d, cfg.num_heads)
        self.ffn = MLP(d, cfg.ffn_dim)

    def forward(self, x, ctx, temb6, rope, sp=None):
        mod = (self.mod_table.unsqueeze(0).float() + temb6.float()).to(x.dtype)  # [B, 6, D]
        m = mod.unbind(1)
        x = self.self_attn(norm_ops.adaln_layernorm(x, m[0], m[1]), rope, m[2], x, sp)
        x = self.cross_attn(self.cross_norm(x), ctx, x)
        return self.ffn(norm_ops.adaln_layernorm(x, m[3], m[4]), gate=m[5], residual=x)


class WanDiT(AdapterMixin, nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.hidden_size
        pt, ph, pw = cfg.patch_size
        in_feats = (cfg.in_channels + cfg.extra_in_channels) * pt * ph * pw
        self.patch_embed = Linear(in_feats, d)
        self.time_embed = TimestepEmbedder(d, cfg.freq_dim)
        self.time_proj = Linear(d, 6 * d, init_std=0.02)
        self.text_embed = MLP(cfg.text_dim, d)
        self.text_embed.fc2 = Linear(d, d)
        self.blocks = nn.ModuleList(WanBlock(cfg) for _ in range(cfg.num_layers))
        self.head_table = nn.Parameter(torch.randn(2, d) / d**0.5)
        self.head = Linear(d, cfg.out_channels * pt * ph * pw, init_std=0.02)
        self.gradient_checkpointing = False
        self._rope_cache: dict = {}

    def enable_gradient_checkpointing(self, flag: bool = True) -> None:
        self.gradient_checkpointing = flag

    def patchify(self, x):
        b, c, f, h, w = x.shape
        pt, ph, pw = self.cfg.patch_size
        grid = (f // pt, h // ph, w // pw)
        x = x.view(b, c, grid[0], pt, grid[1], ph, grid[2], pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(b, grid[0] * grid[1] * grid[2], c * pt * ph * pw), grid

    def unpatchify(self, x, grid):
        b = x.shape[0]
        pt, ph, pw = self.cfg.patch_size
        c = self.cfg.out_channels
        x = x.view(b, *grid, c, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return x.reshape(b, c, grid[0] * pt, grid[1] * ph, grid[2] * pw)

    def rope(self, grid, device):
        key = (grid, str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = rope_3d_tables(
                grid, self.cfg.hidden_size // self.cfg.num_heads, self.cfg.rope_theta, device)
        return self._rope_cache[key]

    def forward(self, latents, timestep, context, sp=None):
        """``latents[B,C,F,H,W]``, ``timestep[B]``, ``context[B,L,text_dim]`` → velocity."""
        dtype = self.patch_embed.weight.dtype
        tokens, grid = self.patchify(latents.to(dtype))
        cos, sin = self.rope(grid, latents.device)
        if sp is not None:
            tokens = sp.shard_sequence(tokens)
            cos, sin = sp.shard_rows(cos), sp.shard_rows(sin)
        x = self.patch_embed(tokens)
        temb = self.time_embed(timestep, dtype)
        temb6 = self.time_proj(torch.nn.functional.silu(temb)).view(-1, 6, self.cfg.hidden_size)
        ctx = self.text_embed(context.to(dtype))
        for block in self.blocks:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                x = checkpoint(block, x, ctx, temb6, (cos, sin), sp, use_reentrant=False)
            else:
                x = block(x, ctx, temb6, (cos, sin), sp)
        mod = (self.head_table.unsqueeze(0).float() + temb.unsqueeze(1).float()).to(dtype)
        x = self.head(norm_ops.adaln_layernorm(x, mod[:, 0], mod[:, 1]))
        if sp is not None:
            x = sp.gather_sequence(x)
        return self.unpatchify(x, grid)

    def flops_per_sample(self, tokens: int, context_tokens: int) -> float:
        cfg = self.cfg
        d, f = cfg.hidden_size, cfg.ffn_dim
        per_tok = 2 * (4 * d * d + 2 * d * d + 2 * d * f)   # self qkv+out, cross q+out, ffn
        ctx = 2 * (2 * d * d) * context_tokens
        attn = 4 * tokens * tokens * d + 4 * tokens * context_tokens * d
        return cfg.num_layers * (per_tok * tokens + ctx + attn)
