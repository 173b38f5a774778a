"""Convolutional latent decoders, a ViT scorer and synthetic text conditioning.

These modules give the frozen parts of a pipeline (VAE / VQ decoder, CLIP-style
reward tower, text encoder) the real shapes and costs with seeded random
weights; checkpoints in the native key layout can be loaded into them with
``load_state_dict``.  Convolutions run in channels-last bf16 through cuDNN.
"""

from __future__ import annotations

import hashlib

import torch
import torch.nn.functional as F
from torch import nn

from visionrl_b200.ops import norm as norm_ops
from visionrl_b200.models.nn.layers import LayerNorm, Linear, MLP, merge_heads, sdpa, split_heads


def _groups(ch: int) -> int:
    for g in (32, 16, 8, 4, 2, 1):
        if ch % g == 0:
            return g
    return 1


class ResBlock2D(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.n1 = nn.GroupNorm(_groups(cin), cin, eps=1e-6)
        self.c1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.n2 = nn.GroupNorm(_groups(cout), cout, eps=1e-6)
        self.c2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.c1(norm_ops.group_norm_silu(x, self.n1))
        h = self.c2(norm_ops.group_norm_silu(h, self.n2))
        return (x if self.skip is None else self.skip(x)) + h


class LatentDecoder2D(nn.Module):
    """``[B, C, h, w]`` latents → ``[B, 3, h*2^k, w*2^k]`` images in ``[-1, 1]``."""

    def __init__(self, in_channels: int = 16, base: int = 128, mults=(1, 2, 4, 4),
                 blocks: int = 2, scaling_factor: float = 1.5305, shift_factor: float = 0.0609):
        super().__init__()
        self.scaling_factor, self.shift_factor = scaling_factor, shift_factor
        top = base * mults[-1]
        self.conv_in = nn.Conv2d(in_channels, top, 3, padding=1)
        self.mid = nn.Sequential(ResBlock2D(top, top), ResBlock2D(top, top))
        stages = []
        ch = top
        for i, m in enumerate(reversed(mults)):
            layers = []
            for _ in range(blocks):
                layers.append(ResBlock2D(ch, base * m))
                ch = base * m
            if i < len(mults) - 1:
                layers.append(nn.Upsample(scale_factor=2.0, mode="nearest"))
                layers.append(nn.Conv2d(ch, ch, 3, padding=1))
            stages.append(nn.Sequential(*layers))
        self.up = nn.Sequential(*stages)
        self.norm_out = nn.GroupNorm(_groups(ch), ch, eps=1e-6)
        self.conv_out = nn.Conv2d(ch, 3, 3, padding=1)
        self.upscale = 2 ** (len(mults) - 1)

    def forward(self, z):
        dtype = self.conv_in.weight.dtype
        z = (z.to(dtype) / self.scaling_factor + self.shift_factor)
        if z.is_cuda:
            z = z.contiguous(memory_format=torch.channels_last)
        h = self.up(self.mid(self.conv_in(z)))
        return self.conv_out(norm_ops.group_norm_silu(h, self.norm_out))


class LatentDecoder3D(nn.Module):
    """Video latents ``[B, C, f, h, w]`` → ``[B, 3, (f-1)*ts+1, H, W]``: frames are decoded
    by a shared 2-D decoder, time is upsampled by linear interpolation."""

    def __init__(self, in_channels: int = 16, base: int = 96, mults=(1, 2, 4, 4), blocks: int = 2,
                 temporal_scale: int = 4):
        super().__init__()
        self.frame_decoder = LatentDecoder2D(in_channels, base, mults, blocks, 1.0, 0.0)
        self.temporal_scale = temporal_scale
        self.register_buffer("latents_mean", torch.zeros(in_channels), persistent=True)
        self.register_buffer("latents_std", torch.ones(in_channels), persistent=True)

    def forward(self, z, frame_chunk: int = 8):
        b, c, f, h, w = z.shape
        z = z.float() * self.latents_std.view(1, c, 1, 1, 1) + self.latents_mean.view(1, c, 1, 1, 1)
        frames = z.permute(0, 2, 1, 3, 4).reshape(b * f, c, h, w)
        out = torch.cat([self.frame_decoder(frames[i:i + frame_chunk])
                         for i in range(0, b * f, frame_chunk)], dim=0)
        out = out.view(b, f, 3, out.shape[-2], out.shape[-1]).permute(0, 2, 1, 3, 4)
        target = (f - 1) * self.temporal_scale + 1
        if target != f:
            out = F.interpolate(out.float(), size=(target, out.shape[-2], out.shape[-1]),
                                mode="trilinear", align_corners=True).to(out.dtype)
        return out


class VQDecoder(nn.Module):
    """Codebook lookup + convolutional decoder (``decode_code`` of a VQ tokenizer)."""

    def __init__(self, codebook_size: int = 16384, codebook_dim: int = 8, base: int = 128,
                 mults=(1, 1, 2, 2, 4), blocks: int = 2):
        super().__init__()
        self.quantize = nn.Module()
        self.quantize.embedding = nn.Embedding(codebook_size, codebook_dim)
        self.decoder = LatentDecoder2D(codebook_dim, base, mults, blocks, 1.0, 0.0)

    @property
    def codebook_dim(self) -> int:
        return int(self.quantize.embedding.weight.shape[-1])

    def decode_code(self, code, shape):
        """``code[B, h*w]`` ids, ``shape=(B, C, h, w)`` → images (unclamped)."""
        b, c, h, w = shape
        z = self.quantize.embedding(code.reshape(b, h, w)).permute(0, 3, 1, 2)
        return self.decoder(z)


VIT_ACTIVATIONS = ("gelu_tanh", "quick_gelu", "gelu")


class ViTBlock(nn.Module):
    """Pre-norm transformer block.  ``act``: ``gelu_tanh`` (fused into the first MLP product;
    what the seeded random towers use), ``quick_gelu`` (``x * sigmoid(1.702 x)``, the OpenAI CLIP
    checkpoints) or ``gelu`` (exact, the OpenCLIP ones)."""

    def __init__(self, dim: int, heads: int, mlp: int, act: str = "gelu_tanh", causal: bool = False):
        super().__init__()
        if act not in VIT_ACTIVATIONS:
            raise ValueError(f"unknown ViT activation {act!r}; expected one of {VIT_ACTIVATIONS}")
        self.heads, self.act, self.causal = heads, act, causal
        self.n1, self.n2 = LayerNorm(dim), LayerNorm(dim)
        self.qkv, self.out = Linear(dim, 3 * dim), Linear(dim, dim)
        self.mlp = MLP(dim, mlp, act="gelu_tanh")

    def _mlp(self, x):
        if self.act == "gelu_tanh":
            return self.mlp(x)
        h = self.mlp.fc1(x)
        h = h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else F.gelu(h)
        return self.mlp.fc2(h)

    def forward(self, x):
        q, k, v = self.qkv(self.n1(x)).chunk(3, dim=-1)
        o = sdpa(*(split_heads(t.contiguous(), self.heads) for t in (q, k, v)), causal=self.causal)
        x = x + self.out(merge_heads(o))
        return x + self._mlp(self.n2(x))


class ViTScorer(nn.Module):
    """ViT image tower with a pooled feature output and a scalar head.

    ``vit_l14`` = 24 layers, 1024 wide, 16 heads, patch 14, 224 px;
    ``vit_b16`` = 12 layers, 768 wide, 12 heads, patch 16, 224 px.
    """

    PRESETS = {
        "vit_l14": dict(layers=24, dim=1024, heads=16, mlp=4096, patch=14, image=224, out_dim=768),
        "vit_b16": dict(layers=12, dim=768, heads=12, mlp=3072, patch=16, image=224, out_dim=512),
        "vit_tiny": dict(layers=2, dim=32, heads=2, mlp=64, patch=8, image=32, out_dim=16),
    }

    def __init__(self, layers=24, dim=1024, heads=16, mlp=4096, patch=14, image=224, out_dim=768,
                 act: str = "gelu_tanh"):
        super().__init__()
        self.patch, self.image, self.act = patch, image, act
        n = (image // patch) ** 2
        self.patch_embed = Linear(3 * patch * patch, dim, bias=False)
        self.cls = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos = nn.Parameter(torch.randn(1, n + 1, dim) * 0.02)
        self.pre_norm, self.post_norm = LayerNorm(dim), LayerNorm(dim)
        self.blocks = nn.ModuleList(ViTBlock(dim, heads, mlp, act) for _ in range(layers))
        self.proj = Linear(dim, out_dim, bias=False)
        self.score_head = Linear(out_dim, 1)
        self.register_buffer("mean", torch.tensor([0.4815, 0.4578, 0.4082]).view(1, 3, 1, 1))
        self.register_buffer("std", torch.tensor([0.2686, 0.2613, 0.2758]).view(1, 3, 1, 1))

    @classmethod
    def from_preset(cls, name: str, act: str = "gelu_tanh") -> "ViTScorer":
        return cls(**cls.PRESETS[name], act=act)

    def features(self, images01):
        """``images01[B,3,H,W]`` in ``[0,1]`` → L2-normalised features ``[B, out_dim]``."""
        dtype = self.patch_embed.weight.dtype
        x = images01.float()
        if x.shape[-2:] != (self.image, self.image):
            x = F.interpolate(x, size=(self.image, self.image), mode="bilinear",
                              align_corners=False, antialias=True)
        x = ((x - self.mean) / self.std).to(dtype)
        b, p, g = x.shape[0], self.patch, self.image // self.patch
        x = x.view(b, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(b, g * g, 3 * p * p)
        x = torch.cat([self.cls.to(dtype).expand(b, -1, -1), self.patch_embed(x)], dim=1)
        x = self.pre_norm(x + self.pos.to(dtype))
        for blk in self.blocks:
            x = blk(x)
        feat = self.proj(self.post_norm(x[:, 0])).float()
        return feat / feat.norm(dim=-1, keepdim=True).clamp_min(1e-6)

    def forward(self, images01):
        return self.score_head(self.features(images01).to(self.score_head.weight.dtype)).float().squeeze(-1)


class CLIPTextTower(nn.Module):
    """Text side of a CLIP checkpoint: token + position embeddings, causal pre-norm blocks, final
    norm, the state at the end-of-text token projected into the joint space and L2-normalised.
    ``eos_token_id=None`` takes the position of the largest token id of each row (end-of-text is
    the last entry of the CLIP vocabulary), otherwise the first occurrence of that id."""

    def __init__(self, layers=12, dim=768, heads=12, mlp=3072, vocab=49408, context=77, out_dim=768,
                 act: str = "quick_gelu", eos_token_id: int | None = None):
        super().__init__()
        self.context, self.eos_token_id = context, eos_token_id
        self.token_embed = nn.Embedding(vocab, dim)
        self.pos = nn.Parameter(torch.randn(context, dim) * 0.01)
        self.blocks = nn.ModuleList(ViTBlock(dim, heads, mlp, act, causal=True) for _ in range(layers))
        self.final_norm = LayerNorm(dim)
        self.proj = Linear(dim, out_dim, bias=False)

    def encode(self, input_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``(penultimate, pooled)``: the output of the second-to-last block ``[B, S, dim]`` (what
        diffusion pipelines condition on) and the projected end-of-text state ``[B, out_dim]``,
        not normalised."""
        b, s = input_ids.shape
        if s > self.context:
            raise ValueError(f"{s} tokens exceed the tower's context of {self.context}")
        dtype = self.proj.weight.dtype
        x = (self.token_embed(input_ids) + self.pos[:s]).to(dtype)
        penultimate = x
        for i, blk in enumerate(self.blocks):
            if i == len(self.blocks) - 1:
                penultimate = x
            x = blk(x)
        x = self.final_norm(x)
        if self.eos_token_id is None:
            last = input_ids.argmax(dim=-1)
        else:
            last = (input_ids == self.eos_token_id).int().argmax(dim=-1)
        return penultimate, self.proj(x[torch.arange(b, device=x.device), last])

    def features(self, input_ids: torch.Tensor) -> torch.Tensor:
        feat = self.encode(input_ids)[1].float()
        return feat / feat.norm(dim=-1, keepdim=True).clamp_min(1e-6)


def _seed_from_text(text: str, salt: str = "") -> int:
    digest = hashlib.sha256((salt + "\x00" + text).encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


class SyntheticTextEncoder:
    """Deterministic stand-in for T5/CLIP text towers: every prompt maps to seeded
    ``N(0, 1)`` token embeddings ``[L, context_dim]`` and a pooled vector.

    Embeddings are generated once into (pinned, when CUDA is present) host memory and copied
    to the device on demand; a per-device cache avoids repeated copies.  ``h2d_bytes`` counts
    the bytes moved since :meth:`reset_transfer_stats`.
    """

    def __init__(self, context_dim: int, pooled_dim: int = 0, salt: str = "text"):
        self.context_dim, self.pooled_dim, self.salt = context_dim, pooled_dim, salt
        self._host: dict = {}
        self._device: dict = {}
        self.h2d_bytes = 0

    def reset_transfer_stats(self) -> None:
        self.h2d_bytes = 0

    def drop_device_cache(self) -> None:
        self._device.clear()

    def _host_entry(self, prompt: str, length: int, dtype):
        key = (prompt, length, dtype)
        if key not in self._host:
            g = torch.Generator().manual_seed(_seed_from_text(prompt, self.salt))
            c = torch.randn(length, self.context_dim, generator=g).to(dtype)
            v = torch.randn(max(self.pooled_dim, 1), generator=g).to(dtype)
            if torch.cuda.is_available():
                c, v = c.pin_memory(), v.pin_memory()
            self._host[key] = (c, v)
        return self._host[key]

    def __call__(self, prompts, length: int, device, dtype):
        if isinstance(prompts, str):
            prompts = [prompts]
        device = torch.device(device)
        ctx, pooled = [], []
        for p in prompts:
            key = (p, length, dtype, str(device))
            if key not in self._device:
                c, v = self._host_entry(p, length, dtype)
                if device.type == "cuda":
                    self.h2d_bytes += c.numel() * c.element_size() + v.numel() * v.element_size()
                    c, v = c.to(device, non_blocking=True), v.to(device, non_blocking=True)
                self._device[key] = (c, v)
            c, v = self._device[key]
            ctx.append(c)
            pooled.append(v)
        ctx_t = torch.stack(ctx)
        pooled_t = torch.stack(pooled) if self.pooled_dim else None
        return ctx_t, pooled_t


class HashTokenizer:
    """Deterministic tokenizer: ids are a seeded function of each character window.

    ``encode`` returns ``max_length`` ids (right-padded with ``pad_id``) and a mask.
    """

    def __init__(self, vocab_size: int, pad_id: int = 0, salt: str = "tok"):
        self.vocab_size, self.pad_id, self.salt = vocab_size, pad_id, salt

    def encode(self, text: str, max_length: int):
        words = text.split() or [""]
        ids = [1 + _seed_from_text(w, self.salt) % (self.vocab_size - 1) for w in words][:max_length]
        mask = [1] * len(ids) + [0] * (max_length - len(ids))
        ids = ids + [self.pad_id] * (max_length - len(ids))
        return ids, mask

    def batch_encode(self, texts, max_length: int, device=None):
        rows = [self.encode(t, max_length) for t in texts]
        ids = torch.tensor([r[0] for r in rows], dtype=torch.long, device=device)
        mask = torch.tensor([r[1] for r in rows], dtype=torch.long, device=device)
        return ids, mask
