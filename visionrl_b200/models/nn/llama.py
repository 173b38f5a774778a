"""LLaMA-style decoder (RMSNorm, rotary attention, SwiGLU) with a static KV cache.

Two entry points share the weights:

* :meth:`LlamaDecoder.forward` — full-sequence causal pass over input embeddings
  (prefill and teacher-forced training replay);
* :meth:`LlamaDecoder.decode_step` — one new position per row against a
  preallocated ``[layers, 2, rows, heads, max_len, head_dim]`` cache, the shape
  the decode-attention kernel (K8) and the int4 weight-only GEMV (K9) consume.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn
from torch.utils.checkpoint import checkpoint

from visionrl_b200.models.nn.layers import (
    AdapterMixin, Linear, LoRALinear, RMSNorm, merge_heads,
)
from visionrl_b200.ops import attention as attn_ops
from visionrl_b200.ops.qkv import apply_rope_reference


@dataclass
class LlamaConfig:
    num_layers: int = 24
    hidden_size: int = 2048
    num_heads: int = 16
    ffn_dim: int = 5632
    vocab_size: int = 102400
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    max_positions: int = 4096
    num_kv_heads: int | None = None     # fewer key/value heads than query heads (grouped-query attention)
    qkv_bias: bool = False              # bias on the fused q/k/v projection (Qwen2-style trunks)

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: d[k] for k in keys if k in d})


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """``positions[...]`` → ``(cos, sin)`` of shape ``[..., head_dim/2]`` (fp32)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32,
                                        device=positions.device) / head_dim))
    ang = positions.float().unsqueeze(-1) * inv
    return torch.cos(ang), torch.sin(ang)


class KVCache:
    """Static key/value storage for ``rows`` sequences of at most ``max_len`` positions."""

    def __init__(self, layers: int, rows: int, heads: int, max_len: int, head_dim: int, device,
                 dtype):
        self.data = torch.zeros(layers, 2, rows, heads, max_len, head_dim, device=device,
                                dtype=dtype)
        self.valid = torch.zeros(rows, max_len, dtype=torch.bool, device=device)
        self.length = 0
        self.max_len = max_len

    def rows(self) -> int:
        return self.data.shape[2]


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.heads, self.head_dim = cfg.num_heads, cfg.hidden_size // cfg.num_heads
        self.kv_heads = int(cfg.num_kv_heads or cfg.num_heads)
        if self.heads % self.kv_heads:
            raise ValueError(f"num_heads={self.heads} is not a multiple of num_kv_heads={self.kv_heads}")
        self.qkv = LoRALinear(cfg.hidden_size, (self.heads + 2 * self.kv_heads) * self.head_dim,
                              bias=bool(cfg.qkv_bias))
        self.out = LoRALinear(cfg.hidden_size, cfg.hidden_size, bias=False)
        self.qkv.lora_aliases = ("q_proj", "k_proj", "v_proj")
        self.out.lora_aliases = ("o_proj",)

    @property
    def plain_layout(self) -> bool:
        """Equal head counts and no bias: the layout the fused decode kernels are written for."""
        return self.kv_heads == self.heads and self.qkv.bias is None

    def _split(self, x):
        b, s, _ = x.shape
        if self.kv_heads == self.heads:
            q, k, v = x.view(b, s, 3, self.heads, self.head_dim).unbind(2)
            return (t.transpose(1, 2) for t in (q, k, v))
        # grouped-query attention: [q | k | v] with fewer k/v heads; every k/v head serves a run of
        # consecutive query heads and is repeated here, so everything downstream (rotary embedding,
        # the cache, the attention calls) sees equal head counts
        hd, group = self.head_dim, self.heads // self.kv_heads
        q, k, v = x.split((self.heads * hd, self.kv_heads * hd, self.kv_heads * hd), dim=-1)
        q = q.view(b, s, self.heads, hd).transpose(1, 2)
        k = k.view(b, s, self.kv_heads, hd).transpose(1, 2).repeat_interleave(group, dim=1)
        v = v.view(b, s, self.kv_heads, hd).transpose(1, 2).repeat_interleave(group, dim=1)
        return iter((q, k, v))


class LlamaLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.attn = LlamaAttention(cfg)
        self.mlp_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.gate_up = Linear(cfg.hidden_size, 2 * cfg.ffn_dim, bias=False)
        self.down = Linear(cfg.ffn_dim, cfg.hidden_size, bias=False)

    def mlp(self, x):
        g, u = self.gate_up(x).chunk(2, dim=-1)
        return self.down(F.silu(g) * u)

    def forward(self, x, cos, sin, bias, cache=None, layer_idx: int = 0, start: int = 0):
        q, k, v = self.attn._split(self.attn.qkv(self.attn_norm(x)))
        q = apply_rope_reference(q, cos, sin)
        k = apply_rope_reference(k, cos, sin)
        if cache is not None:
            s = k.shape[2]
            cache.data[layer_idx, 0, :, :, start:start + s] = k
            cache.data[layer_idx, 1, :, :, start:start + s] = v
        if bias is None:
            o = attn_ops.attention(q, k, v, causal=True)
        else:
            o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        x = x + self.attn.out(merge_heads(o))
        return x + self.mlp(self.mlp_norm(x))

    def decode_at(self, x, cos, sin, cache: KVCache, layer_idx: int, pos: torch.Tensor):
        """:meth:`decode` for all rows with the position as a device tensor (graph-capturable)."""
        q, k, v = self.attn._split(self.attn.qkv(self.attn_norm(x)))
        q = apply_rope_reference(q, cos, sin)
        k = apply_rope_reference(k, cos, sin)
        cache.data[layer_idx, 0].index_copy_(2, pos, k)
        cache.data[layer_idx, 1].index_copy_(2, pos, v.contiguous())
        o = attn_ops.decode_attention(q, cache.data[layer_idx, 0], cache.data[layer_idx, 1],
                                      cache.valid, cache.max_len)
        x = x + self.attn.out(merge_heads(o))
        return x + self.mlp(self.mlp_norm(x))

    def decode(self, x, cos, sin, cache: KVCache, layer_idx: int, rows=None, pos=None):
        """``x[R, 1, D]`` at position ``pos`` (already marked valid) of cache rows ``rows``."""
        q, k, v = self.attn._split(self.attn.qkv(self.attn_norm(x)))
        q = apply_rope_reference(q, cos, sin)
        k = apply_rope_reference(k, cos, sin)
        pos = cache.length if pos is None else pos
        if rows is None:
            cache.data[layer_idx, 0, :, :, pos] = k[:, :, 0]
            cache.data[layer_idx, 1, :, :, pos] = v[:, :, 0]
            o = attn_ops.decode_attention(q, cache.data[layer_idx, 0], cache.data[layer_idx, 1],
                                          cache.valid, pos + 1)
        else:
            cache.data[layer_idx, 0, rows, :, pos] = k[:, :, 0]
            cache.data[layer_idx, 1, rows, :, pos] = v[:, :, 0]
            o = attn_ops.decode_attention_reference(
                q, cache.data[layer_idx, 0][rows], cache.data[layer_idx, 1][rows],
                cache.valid[rows], pos + 1)
        x = x + self.attn.out(merge_heads(o))
        return x + self.mlp(self.mlp_norm(x))


class LlamaDecoder(AdapterMixin, nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        nn.init.normal_(self.embed_tokens.weight, std=0.02)
        self.layers = nn.ModuleList(LlamaLayer(cfg) for _ in range(cfg.num_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.gradient_checkpointing = False

    @property
    def head_dim(self) -> int:
        return self.cfg.hidden_size // self.cfg.num_heads

    def new_cache(self, rows: int, max_len: int, device=None, dtype=None) -> KVCache:
        w = self.embed_tokens.weight
        return KVCache(self.cfg.num_layers, rows, self.cfg.num_heads, max_len, self.head_dim,
                       device or w.device, dtype or w.dtype)

    def forward(self, embeds, attention_mask=None, cache: KVCache | None = None):
        """``embeds[B, S, D]``; ``attention_mask[B, S]`` marks real (1) vs padded (0) keys."""
        b, s, _ = embeds.shape
        pos = torch.arange(s, device=embeds.device)
        cos, sin = rope_tables(pos, self.head_dim, self.cfg.rope_theta)
        bias = None
        if attention_mask is not None and not bool(attention_mask.all()):
            causal = torch.ones(s, s, dtype=torch.bool, device=embeds.device).tril()
            keep = causal[None, None] & attention_mask.bool()[:, None, None, :]
            keep = keep | torch.eye(s, dtype=torch.bool, device=embeds.device)[None, None]
            bias = torch.zeros(b, 1, s, s, dtype=embeds.dtype, device=embeds.device)
            bias.masked_fill_(~keep, float("-inf"))
        if cache is not None:
            cache.valid[:, :s] = True if attention_mask is None else attention_mask.bool()
            cache.length = s
        x = embeds
        for i, layer in enumerate(self.layers):
            if self.gradient_checkpointing and torch.is_grad_enabled() and cache is None:
                x = checkpoint(layer, x, cos, sin, bias, use_reentrant=False)
            else:
                x = layer(x, cos, sin, bias, cache, i, 0)
        return self.norm(x)

    def decode_step_at(self, embeds, cache: KVCache, pos: torch.Tensor):
        """One decode step of every cache row at the position held in the device tensor ``pos``
        (int64, one element).

        Nothing here depends on a host-side value: the cache is written with ``index_copy_``,
        the rotary angles are computed from ``pos`` and attention walks the whole static cache
        with the validity mask selecting the filled positions.  The step can therefore be
        captured once in a CUDA graph and replayed for every position; the caller keeps
        ``cache.length`` up to date.
        """
        cache.valid.index_fill_(1, pos, True)
        cos, sin = rope_tables(pos, self.head_dim, self.cfg.rope_theta)
        if self._fused_decode_ok(embeds):
            return self._decode_step_fused(embeds, cache, pos, cos, sin)
        x = embeds.unsqueeze(1)
        for i, layer in enumerate(self.layers):
            x = layer.decode_at(x, cos, sin, cache, i, pos)
        return self.norm(x)[:, 0]

    def _fused_decode_ok(self, embeds) -> bool:
        from visionrl_b200.ops import _ext

        return (embeds.is_cuda and embeds.dtype == torch.bfloat16 and embeds.dim() == 2
                and self.layers[0].attn.plain_layout
                and not torch.is_grad_enabled() and self.head_dim == 128
                and self.cfg.hidden_size % 8 == 0 and self.cfg.ffn_dim % 8 == 0
                and _ext.kernels_enabled() and _ext.has("decode_qkv_rope_append"))

    def _decode_step_fused(self, embeds, cache: KVCache, pos, cos, sin):
        """The decode step with its glue folded into three kernels per layer: residual add + RMSNorm,
        RoPE + cache append on the QKV output, SwiGLU.  A layer is then 13 launches (four
        projections of two launches each, attention, and the glue) instead of some forty, which
        is what a step of 32 rows — launch latency, not bandwidth — is made of."""
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        rows, d = embeds.shape
        eps = float(self.norm.eps)
        cos1, sin1 = cos.reshape(-1).contiguous(), sin.reshape(-1).contiguous()
        x = embeds.clone()                       # updated in place by the fused residual adds
        delta = None
        heads = self.layers[0].attn.heads

        def weight(norm):
            w = norm.weight
            return w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)

        for i, layer in enumerate(self.layers):
            h = ext.add_rmsnorm_rows(x, delta, weight(layer.attn_norm), float(layer.attn_norm.eps))
            qkv = layer.attn.qkv(h)
            q = ext.decode_qkv_rope_append(qkv.contiguous(), cos1, sin1, pos, cache.data[i, 0],
                                           cache.data[i, 1], heads)
            o = attn_ops.decode_attention(q, cache.data[i, 0], cache.data[i, 1], cache.valid, cache.max_len)
            a = layer.attn.out(o.view(rows, d))
            h2 = ext.add_rmsnorm_rows(x, a.contiguous(), weight(layer.mlp_norm), float(layer.mlp_norm.eps))
            delta = layer.down(ext.swiglu_rows(layer.gate_up(h2).contiguous())).contiguous()
        return ext.add_rmsnorm_rows(x, delta, weight(self.norm), eps)

    def decode_step(self, embeds, cache: KVCache, rows=None, position: int | None = None):
        """``embeds[R, D]`` for the next position → hidden ``[R, D]``.

        Without ``rows`` every cache row advances together from ``cache.length``.  With ``rows``
        (a long tensor) only those rows are stepped, at the explicit ``position``; rows may then
        sit at different lengths, which token-level scheduling needs.
        """
        pos = cache.length if position is None else int(position)
        if pos >= cache.max_len:
            raise RuntimeError(f"KV cache is full ({cache.max_len} positions)")
        if rows is None:
            cache.valid[:, pos] = True
        else:
            cache.valid[rows, pos] = True
        cos, sin = rope_tables(torch.tensor([pos], device=embeds.device), self.head_dim,
                               self.cfg.rope_theta)
        x = embeds.unsqueeze(1)
        for i, layer in enumerate(self.layers):
            x = layer.decode(x, cos, sin, cache, i, rows, pos)
        if rows is None:
            cache.length = pos + 1
        else:
            cache.length = max(cache.length, pos + 1)
        return self.norm(x)[:, 0]
