"""Text encoders of the diffusion families, native: the T5 / UMT5 encoder stack.

The encoder is frozen and runs once per prompt (its output is cached on the host and copied to
the device per step), so it is written with plain library products; its job here is to give the
same numbers as the public implementation from the same weights, which the tests check against
``transformers.T5EncoderModel`` and ``transformers.UMT5EncoderModel``.

T5 specifics kept: attention without the ``1/sqrt(d)`` scale, an additive relative-position bias
looked up from bucketed signed distances (one table shared by all layers in T5, one table per
layer in UMT5), RMS normalisation without bias, a gated feed-forward
(``wo(act(wi_0 x) * wi_1 x)``) with the tanh-approximated GELU.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class T5EncoderConfig:
    vocab_size: int = 256384
    d_model: int = 4096
    d_kv: int = 64
    d_ff: int = 10240
    num_layers: int = 24
    num_heads: int = 64
    num_buckets: int = 32
    max_distance: int = 128
    per_layer_bias: bool = False        # True: UMT5 (every layer owns a bias table)
    gated: bool = True                  # False: the original T5 feed-forward wo(relu(wi x))
    eps: float = 1e-6

    @classmethod
    def from_hf(cls, config: dict) -> "T5EncoderConfig":
        proj = str(config.get("feed_forward_proj", "relu"))
        return cls(vocab_size=int(config["vocab_size"]), d_model=int(config["d_model"]), d_kv=int(config["d_kv"]),
                   d_ff=int(config["d_ff"]), num_layers=int(config["num_layers"]), num_heads=int(config["num_heads"]),
                   num_buckets=int(config.get("relative_attention_num_buckets", 32)),
                   max_distance=int(config.get("relative_attention_max_distance", 128)),
                   per_layer_bias=str(config.get("model_type", "t5")) == "umt5", gated=proj.startswith("gated"),
                   eps=float(config.get("layer_norm_epsilon", 1e-6)))


def relative_position_bucket(relative_position: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional T5 bucketing of ``key_position - query_position``: half of the buckets per
    sign; within a sign, exact buckets for small distances and log-spaced ones up to
    ``max_distance``, everything beyond in the last bucket."""
    half = num_buckets // 2
    bucket = (relative_position > 0).long() * half
    distance = relative_position.abs()
    exact = half // 2
    log_bucket = exact + (torch.log(distance.float().clamp_min(1) / exact) / math.log(max_distance / exact)
                          * (half - exact)).long()
    log_bucket = log_bucket.clamp(max=half - 1)
    return bucket + torch.where(distance < exact, distance, log_bucket)


class T5RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        var = x.float().pow(2).mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(var + self.eps)).to(self.weight.dtype) * self.weight


class T5Block(nn.Module):
    def __init__(self, cfg: T5EncoderConfig, own_bias: bool):
        super().__init__()
        inner = cfg.num_heads * cfg.d_kv
        self.heads, self.d_kv, self.gated = cfg.num_heads, cfg.d_kv, cfg.gated
        self.attn_norm = T5RMSNorm(cfg.d_model, cfg.eps)
        self.q = nn.Linear(cfg.d_model, inner, bias=False)
        self.k = nn.Linear(cfg.d_model, inner, bias=False)
        self.v = nn.Linear(cfg.d_model, inner, bias=False)
        self.o = nn.Linear(inner, cfg.d_model, bias=False)
        self.rel_bias = nn.Embedding(cfg.num_buckets, cfg.num_heads) if own_bias else None
        self.ff_norm = T5RMSNorm(cfg.d_model, cfg.eps)
        self.wi_0 = nn.Linear(cfg.d_model, cfg.d_ff, bias=False)
        self.wi_1 = nn.Linear(cfg.d_model, cfg.d_ff, bias=False) if cfg.gated else None
        self.wo = nn.Linear(cfg.d_ff, cfg.d_model, bias=False)

    def forward(self, x, bias):
        b, s, _ = x.shape
        h = self.attn_norm(x)
        q, k, v = (proj(h).view(b, s, self.heads, self.d_kv).transpose(1, 2) for proj in (self.q, self.k, self.v))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype), scale=1.0)
        x = x + self.o(o.transpose(1, 2).reshape(b, s, -1))
        h = self.ff_norm(x)
        if self.gated:
            h = F.gelu(self.wi_0(h), approximate="tanh") * self.wi_1(h)
        else:
            h = F.relu(self.wi_0(h))
        return x + self.wo(h)


class T5Encoder(nn.Module):
    def __init__(self, cfg: T5EncoderConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList(T5Block(cfg, own_bias=cfg.per_layer_bias or i == 0)
                                    for i in range(cfg.num_layers))
        self.final_norm = T5RMSNorm(cfg.d_model, cfg.eps)

    def _bias(self, table: nn.Embedding, s: int, device) -> torch.Tensor:
        pos = torch.arange(s, device=device)
        buckets = relative_position_bucket(pos[None, :] - pos[:, None], self.cfg.num_buckets, self.cfg.max_distance)
        return table(buckets).permute(2, 0, 1).unsqueeze(0)             # [1, H, S, S]

    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """``input_ids[B, S]`` (and ``attention_mask[B, S]``, 1 = real token) → ``[B, S, d_model]``."""
        b, s = input_ids.shape
        x = self.embed(input_ids)
        pad = None
        if attention_mask is not None:
            pad = torch.zeros(b, 1, 1, s, dtype=torch.float32, device=x.device)
            pad.masked_fill_(~attention_mask.bool()[:, None, None, :], torch.finfo(torch.float32).min)
        shared = None
        for blk in self.blocks:
            if blk.rel_bias is not None:
                shared = self._bias(blk.rel_bias, s, x.device).float()
            bias = shared if pad is None else shared + pad
            x = blk(x, bias)
        return self.final_norm(x)


__all__ = ["T5Block", "T5Encoder", "T5EncoderConfig", "T5RMSNorm", "relative_position_bucket"]
