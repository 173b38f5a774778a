"""NextStep-1-style continuous-token autoregressive policy.

A LLaMA/Qwen-style trunk consumes text tokens followed by continuous image tokens (projected by
``image_in``); at every image position the trunk's hidden state conditions a small adaLN MLP
flow head that produces the next ``token_dim``-channel token by flow matching
(:mod:`.flow_step`).  Rollout records the token, its Gaussian log-probability and the prior
noise ``x_0``; the replay teacher-forces the recorded tokens through the trunk in one pass and
re-integrates the head with the saved ``x_0`` (reference:
``vrl/models/families/nextstep_1/policy.py:137-702``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterator

import torch
from torch import nn

from visionrl_b200.models.ar import ARStepResult
from visionrl_b200.models.families.flow_policy import resolve_dtype, seeded_construction, seeded_init
from visionrl_b200.models.families.nextstep_1.flow_step import (
    flow_logprob_at, flow_sample_with_logprob,
)
from visionrl_b200.models.nn.layers import (
    Linear, adapters_disabled, apply_lora, iter_lora_layers, timestep_embedding,
)
from visionrl_b200.models.nn.llama import KVCache, LlamaConfig, LlamaDecoder
from visionrl_b200.models.nn.vision import HashTokenizer, LatentDecoder2D
from visionrl_b200.ops import norm as norm_ops


# the published model's continuous-token geometry (defaults of the config below)
NEXTSTEP_DEFAULT_TOKEN_NUM = 1024
NEXTSTEP_DEFAULT_TOKEN_DIM = 64
NEXTSTEP_DEFAULT_PIXEL_SIZE = 256


@dataclass
class NextStep1Config:
    model_path: str = "stepfun-ai/NextStep-1.1"
    vae_path: str = "stepfun-ai/NextStep-1-f8ch16-Tokenizer"
    dtype: str = "bfloat16"
    use_lora: bool = True
    lora_rank: int = 32
    lora_alpha: int = 64
    lora_dropout: float = 0.0
    lora_init: str = "gaussian"
    lora_target_modules: tuple = ("q_proj", "k_proj", "v_proj", "o_proj")
    cfg_scale: float = 4.5
    num_flow_steps: int = 20
    noise_level: float = 1.0
    image_token_num: int = 1024
    image_size: int = 256
    freeze_image_head: bool = False
    random_init: bool = True
    init_seed: int = 0
    arch: dict = field(default_factory=dict)
    # fields of the reference's config, accepted so that code and YAML written for it construct this one
    device: str | None = None
    token_dim: int | None = None                # overrides arch["token_dim"] when set
    freeze_vae: bool = True                     # the decoder is always frozen here
    gradient_checkpointing: bool = False        # recompute the trunk's blocks in backward


class FlowHeadBlock(nn.Module):
    def __init__(self, width: int):
        super().__init__()
        self.mod = Linear(width, 3 * width, init_std=0.02)
        self.fc1 = Linear(width, width)
        self.fc2 = Linear(width, width)

    def forward(self, h, c_act):
        shift, scale, gate = self.mod(c_act).chunk(3, dim=-1)
        y = norm_ops.adaln_layernorm(h.unsqueeze(1), shift, scale).squeeze(1)
        return h + gate * self.fc2(self.fc1(y, act="silu"))


class FlowHeadNet(nn.Module):
    """adaLN MLP velocity field ``v(x, t, cond)``."""

    def __init__(self, token_dim: int, cond_dim: int, width: int, layers: int):
        super().__init__()
        self.width = width
        self.x_in = Linear(token_dim, width)
        self.t_in = Linear(256, width)
        self.c_in = Linear(cond_dim, width)
        self.blocks = nn.ModuleList(FlowHeadBlock(width) for _ in range(layers))
        self.out_mod = Linear(width, 2 * width, init_std=0.02)
        self.out = Linear(width, token_dim, init_std=0.02)

    def forward(self, x, t, cond):
        dtype = self.x_in.weight.dtype
        c = self.t_in(timestep_embedding(t * 1000.0, 256).to(dtype)) + self.c_in(cond.to(dtype))
        c_act = torch.nn.functional.silu(c)
        h = self.x_in(x.to(dtype))
        for blk in self.blocks:
            h = blk(h, c_act)
        shift, scale = self.out_mod(c_act).chunk(2, dim=-1)
        y = norm_ops.adaln_layernorm(h.unsqueeze(1), shift, scale).squeeze(1)
        return self.out(y).to(x.dtype)


class FlowMatchingHead(nn.Module):
    def __init__(self, token_dim: int, cond_dim: int, width: int, layers: int):
        super().__init__()
        self.input_dim = token_dim
        self.net = FlowHeadNet(token_dim, cond_dim, width, layers)


class NextStepNetwork(nn.Module):
    def __init__(self, arch: dict[str, Any]):
        super().__init__()
        cfg = LlamaConfig.from_dict(arch)
        token_dim = int(arch.get("token_dim", 64))
        self.language_model = LlamaDecoder(cfg)
        self.image_in = Linear(token_dim, cfg.hidden_size)
        self.image_head = FlowMatchingHead(token_dim, cfg.hidden_size,
                                           int(arch.get("head_hidden", 1536)),
                                           int(arch.get("head_layers", 12)))


@dataclass
class NextStep1ARState:
    cache: KVCache
    tokens: torch.Tensor         # [B, L, D]
    log_probs: torch.Tensor      # [B, L]
    saved_noise: torch.Tensor    # [B, L, D]  prior x_0 per token
    final_noise: torch.Tensor    # [B, L, D]  last-step eps per token
    last_hidden: torch.Tensor    # [2B, H]
    positions: torch.Tensor
    text_len: int
    cfg_scale: float
    num_flow_steps: int
    noise_level: float
    image_token_num: int


class NextStep1Policy(nn.Module):
    family = "nextstep_1"
    model_family = "nextstep_1"

    def __init__(self, config: NextStep1Config | None = None, *, network: NextStepNetwork | None = None,
                 vae: nn.Module | None = None, device: Any = "cpu") -> None:
        super().__init__()
        self.config = config or NextStep1Config()
        arch = dict(self.config.arch)
        if self.config.token_dim is not None:
            arch["token_dim"] = int(self.config.token_dim)
        dtype = resolve_dtype(self.config.dtype)
        if self.config.device is not None and str(device) == "cpu":
            device = self.config.device          # the reference names the device in the config
        dev = torch.device(device)
        if network is None:
            if not self.config.random_init:
                raise FileNotFoundError(
                    "checkpoint-backed NextStep loading expects weights in the native key layout; "
                    "set model.random_init=true for seeded random weights")
            with seeded_construction(self.config.init_seed, dev):
                network = NextStepNetwork(arch)
                seeded_init(network, self.config.init_seed)
        self.policy = network.to(device=dev, dtype=dtype)
        if self.config.gradient_checkpointing:
            self.policy.language_model.gradient_checkpointing = True
        self.token_dim = int(self.policy.image_head.input_dim)
        if vae is None:
            patch = int(arch.get("token_patch", 2))
            channels = self.token_dim // (patch * patch)
            with seeded_construction(self.config.init_seed + 1, dev):
                vae = LatentDecoder2D(channels, int(arch.get("vae_base", 64)),
                                      tuple(arch.get("vae_mults", (1, 2, 4))),
                                      int(arch.get("vae_blocks", 1)), 1.0, 0.0)
                seeded_init(vae, self.config.init_seed + 1)
        object.__setattr__(self, "_vae", vae.to(device=dev, dtype=dtype if dev.type == "cuda"
                                                else torch.float32).eval().requires_grad_(False))
        self.tokenizer = HashTokenizer(self.policy.language_model.cfg.vocab_size)
        self.policy.language_model.embed_tokens.requires_grad_(False)
        if self.config.use_lora:
            apply_lora(self.policy.language_model, self.config.lora_rank, self.config.lora_alpha,
                       list(self.config.lora_target_modules), self.config.lora_init)
            self.policy.image_in.requires_grad_(False)
            self.policy.image_head.requires_grad_(not self.config.freeze_image_head)

    # -- access ---------------------------------------------------------------------------
    @property
    def device(self) -> torch.device:
        return self.policy.image_in.weight.device

    @property
    def dtype(self) -> torch.dtype:
        return self.policy.image_in.weight.dtype

    @property
    def language_model(self) -> LlamaDecoder:
        return self.policy.language_model

    @property
    def trainable_modules(self) -> dict[str, Any]:
        return {"policy": self.policy}

    def trainable_param_count(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    @property
    def has_adapters(self) -> bool:
        return any(True for _ in iter_lora_layers(self.policy.language_model))

    def disable_adapter(self):
        if not self.has_adapters:
            raise RuntimeError("NextStep1Policy.disable_adapter(): the trunk carries no adapter")
        return adapters_disabled(self.policy.language_model)

    def load_trainable_state(self, state_dict: dict[str, Any]) -> Any:
        state = dict(state_dict)
        if not state:
            raise ValueError("load_trainable_state received an empty state dict")
        bad = [k for k in state if not k.startswith("policy.")]
        if bad:
            raise ValueError(f"load_trainable_state only accepts 'policy.'-prefixed keys; got {bad[:4]}")
        return self.policy.load_state_dict({k[7:]: v for k, v in state.items()}, strict=False)

    def embed_text(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.policy.language_model.embed_tokens(token_ids)

    # -- sampling -----------------------------------------------------------------------------
    @torch.no_grad()
    def init_ar_state(self, prompt_embeds, uncond_embeds, prompt_mask, uncond_mask, *, cfg_scale=None,
                      num_flow_steps=None, noise_level=None, image_token_num=None,
                      generator: torch.Generator | None = None) -> NextStep1ARState:
        cond_inputs_embeds, uncond_inputs_embeds = prompt_embeds, uncond_embeds
        cond_attention_mask, uncond_attention_mask = prompt_mask, uncond_mask
        c = self.config
        n_img = int(image_token_num or c.image_token_num)
        b, l_text = cond_attention_mask.shape
        lm = self.policy.language_model
        cache = lm.new_cache(2 * b, l_text + n_img, device=self.device, dtype=self.dtype)
        embeds = torch.cat([cond_inputs_embeds, uncond_inputs_embeds], dim=0).to(self.dtype)
        mask = torch.cat([cond_attention_mask, uncond_attention_mask], dim=0)
        hidden = lm(embeds, mask, cache=cache)
        shape = (b, n_img, self.token_dim)

        def draw():
            if generator is not None and generator.device.type != self.device.type:
                return torch.randn(shape, generator=generator).to(self.device, torch.float32)
            return torch.randn(shape, generator=generator, device=self.device, dtype=torch.float32)

        return NextStep1ARState(
            cache=cache, tokens=torch.zeros(shape, device=self.device, dtype=torch.float32),
            log_probs=torch.zeros(b, n_img, device=self.device, dtype=torch.float32),
            saved_noise=draw(), final_noise=draw(), last_hidden=hidden[:, -1].contiguous(),
            positions=torch.zeros(b, dtype=torch.long, device=self.device), text_len=l_text,
            cfg_scale=float(c.cfg_scale if cfg_scale is None else cfg_scale),
            num_flow_steps=int(num_flow_steps or c.num_flow_steps),
            noise_level=float(c.noise_level if noise_level is None else noise_level),
            image_token_num=n_img)

    def _sample_rows(self, state: NextStep1ARState, rows, position: int):
        b = state.tokens.shape[0]
        idx = torch.arange(b, device=self.device) if rows is None else rows
        cond, uncond = state.last_hidden[idx].float(), state.last_hidden[idx + b].float()
        res = flow_sample_with_logprob(
            self.policy.image_head, cond, num_flow_steps=state.num_flow_steps,
            noise_level=state.noise_level, cfg_uncond=uncond, cfg_scale=state.cfg_scale,
            initial_noise=state.saved_noise[idx, position], final_noise=state.final_noise[idx, position])
        state.tokens[idx, position] = res.token.float()
        state.log_probs[idx, position] = res.log_prob.float()
        if position + 1 < state.image_token_num:
            nxt = self.policy.image_in(res.token.to(self.dtype))
            lm = self.policy.language_model
            both = torch.cat([idx, idx + b])
            if rows is None:
                state.last_hidden = lm.decode_step(torch.cat([nxt, nxt]), state.cache)
            else:
                state.last_hidden[both] = lm.decode_step(torch.cat([nxt, nxt]), state.cache, rows=both,
                                                         position=state.text_len + position)
        state.positions[idx] += 1
        return res.token, res.log_prob

    @torch.no_grad()
    def sample_image_tokens(self, cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                            uncond_attention_mask, **kwargs: Any):
        state = self.init_ar_state(cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                                   uncond_attention_mask, **kwargs)
        for position in range(state.image_token_num):
            self._sample_rows(state, None, position)
        return self.finalize_ar_state(state)

    @torch.no_grad()
    def step_ar(self, state: NextStep1ARState, sequences: list[Any], *,
                generator: torch.Generator | None = None) -> ARStepResult:
        del generator
        if not sequences:
            raise ValueError("step_ar requires at least one ActiveSequence")
        rows = [int(s.metadata.get("row_index", -1)) for s in sequences]
        if any(r < 0 or r >= state.tokens.shape[0] for r in rows):
            raise ValueError(f"invalid NextStep row indices: {rows}")
        positions = {int(s.position) for s in sequences}
        if len(positions) != 1:
            raise ValueError("step_ar requires sequences at one common position")
        position = positions.pop()
        idx = torch.tensor(rows, dtype=torch.long, device=self.device)
        token, log_prob = self._sample_rows(state, idx, position)
        return ARStepResult(sequence_ids=[s.sample_id for s in sequences],
                            positions=[position] * len(sequences), token=token, log_prob=log_prob,
                            replay_extras={"saved_noise": state.saved_noise[idx, position]})

    def finalize_ar_state(self, state: NextStep1ARState):
        """``(tokens, saved_noise, log_probs)`` — the order of the reference's 3-tuple."""
        return state.tokens, state.saved_noise, state.log_probs

    # -- replay -----------------------------------------------------------------------------------
    def recompute_logprobs(self, prompt_embeds, uncond_embeds, prompt_mask, uncond_mask, tokens,
                           saved_noise, *, cfg_scale: float, num_flow_steps: int,
                           noise_level: float) -> torch.Tensor:
        """``[B, L]`` log-probs of recorded ``tokens`` with the rollout's ``x_0`` (exact replay).
        Argument order as in the reference: both embeddings, then both masks."""
        b, l_img, d = tokens.shape
        l_text = prompt_mask.shape[1]
        lm = self.policy.language_model
        img = self.policy.image_in(tokens[:, :-1].to(self.dtype)) if l_img > 1 else \
            prompt_embeds.new_zeros(b, 0, prompt_embeds.shape[-1])

        def hidden_for(embeds, mask):
            seq = torch.cat([embeds.to(self.dtype), img], dim=1)
            full = torch.cat([mask, mask.new_ones(b, l_img - 1)], dim=1)
            return lm(seq, full)[:, l_text - 1: l_text - 1 + l_img]

        cond = hidden_for(prompt_embeds, prompt_mask)
        with torch.no_grad():
            uncond = hidden_for(uncond_embeds, uncond_mask)
        # the final-step noise is implied: token - mu; only x_0 is needed for the mean
        lp = flow_logprob_at(
            self.policy.image_head, cond.reshape(b * l_img, -1).float(),
            tokens.reshape(b * l_img, d).float(), saved_noise.reshape(b * l_img, d).float(),
            num_flow_steps=num_flow_steps, noise_level=noise_level,
            cfg_uncond=uncond.reshape(b * l_img, -1).float(), cfg_scale=cfg_scale)
        return lp.view(b, l_img)

    def replay_forward(self, batch: Any, timestep_idx: int = 0) -> dict[str, Any]:
        obs = batch.observations
        ids = (obs[:, 0] if obs.ndim == 3 else obs).to(self.device)
        ctx = batch.context
        lp = self.recompute_logprobs(
            prompt_embeds=self.embed_text(ids),
            uncond_embeds=self.embed_text(batch.extras["uncond_input_ids"].to(self.device)),
            prompt_mask=batch.extras["prompt_attention_mask"].to(self.device),
            uncond_mask=batch.extras["uncond_attention_mask"].to(self.device), tokens=batch.actions.to(self.device),
            saved_noise=batch.extras["saved_noise"].to(self.device), cfg_scale=float(ctx["cfg_scale"]),
            num_flow_steps=int(ctx["num_flow_steps"]), noise_level=float(ctx["noise_level"]))
        return {"log_probs": lp, "target_tokens": batch.actions}

    # -- decoding -----------------------------------------------------------------------------------
    @torch.no_grad()
    def decode_image_tokens(self, tokens: torch.Tensor, image_size: int | None = None):
        b, n, d = tokens.shape
        side = int(round(n ** 0.5))
        if side * side != n:
            raise ValueError(f"image token count {n} is not a square grid")
        patch = int(round((d // self._vae.conv_in.in_channels) ** 0.5))
        ch = self._vae.conv_in.in_channels
        lat = tokens.view(b, side, side, ch, patch, patch).permute(0, 3, 1, 4, 2, 5)
        lat = lat.reshape(b, ch, side * patch, side * patch)
        images = self._vae(lat).float().clamp(-1.0, 1.0)
        if image_size is not None and images.shape[-1] != image_size:
            images = torch.nn.functional.interpolate(images, size=(image_size, image_size),
                                                     mode="bilinear", align_corners=False)
        return images


__all__ = ["FlowMatchingHead", "NextStep1ARState", "NextStep1Config", "NextStep1Policy",
           "NextStepNetwork"]
